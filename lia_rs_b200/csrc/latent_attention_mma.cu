// Attention in a latent's space on the tensor cores (bfloat16, mma.sync): every query head of a token reads the same
// records of the paged cache, a latent of `rank` elements that is key and value at once, and a rotated key part of `dr`
// elements:
//     score(h, j) = scale * (q1[h] . latent_j + q2[h] . part_j),   out[h] = sum_j softmax_j(score) latent_j
// for the keys j of the token's own request with max(0, pos - window + 1) <= j <= pos.
//
// One CTA serves one token and up to 16 of its heads (the M of an m16n8k16 product) and walks the token's keys 32 at a
// time: the tile's records come into shared memory once for all heads, by asynchronous copies issued a tile ahead;
// warp w multiplies the queries with keys 8w..8w+7
// over all of rank + dr; the scores meet in shared memory; every warp takes the softmax of the 16 x 32 scores for itself
// (32-bit, base 2, running maximum and sum per row) and multiplies the probabilities, rounded to bfloat16, with its own
// quarter of the latent's columns, accumulating in 32-bit registers.  Prompt portions and single tokens are the same
// kernel.  With `splits` > 1 a token's tiles are cut into that many ranges (grid z) that leave unnormalised sums, maxima
// and outputs in scratch, and a second kernel puts them together; the number of ranges is the caller's choice and the
// cut depends on the token's own span alone.
//
// q1 [heads, tokens, rank] and out [heads, tokens, rank] are planes per head (a head's rows are a matrix for the
// products before and after), q2 [tokens, heads, dr].  rank a multiple of 32 up to 512, dr a multiple of 16 up to 128.

#include "common.cuh"

namespace {
constexpr int KEYS = 32;             // keys per tile
constexpr int THREADS = 128;
constexpr int PAD = 8;               // elements added to a shared-memory row: rows then start in different banks
constexpr float LOG2E = 1.4426950408889634f;

struct LatentParams {
    const __nv_bfloat16* q1;
    const __nv_bfloat16* q2;
    const __nv_bfloat16* latent_pages;   // [pages, page_size, rank]
    const __nv_bfloat16* part_pages;     // [pages, page_size, dr]
    const int* positions;
    const int* slots;
    const int* block_table;
    __nv_bfloat16* out;
    float* partial;                      // splits > 1: [splits][heads][tokens][rank] outputs, then [splits][heads][tokens][2] maximum and sum
    int n_tokens, heads, rank, dr, table_stride, page_size, window, num_pages, splits;
    float scale_log2;
    int* error_flag;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int NT>                      // 8-column tiles of the output per warp: rank / 32
__global__ void __launch_bounds__(THREADS)
latent_attention_kernel(LatentParams p) {
    extern __shared__ __align__(16) uint8_t latent_smem[];
    const int dk = p.rank + p.dr, ld = dk + PAD;
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(latent_smem);              // [16][ld]
    __nv_bfloat16* ks_all = qs + 16 * ld;                                             // [2][KEYS][ld]: this tile and the next
    float* ss = reinterpret_cast<float*>(ks_all + 2 * KEYS * ld);                     // [16][KEYS + 1]
    int* key_rows_all = reinterpret_cast<int*>(ss + 16 * (KEYS + 1));                 // [2][KEYS]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h0 = blockIdx.y * 16;
    const int slot = p.slots[t];
    if (slot < 0) return;
    const int pos = p.positions[t];
    const int first = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int n_tiles = (pos - first + KEYS) / KEYS;
    const int per = (n_tiles + p.splits - 1) / p.splits;
    const int tile_lo = blockIdx.z * per, tile_hi = min(n_tiles, tile_lo + per);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int heads_here = min(16, p.heads - h0);
    const int* table = p.block_table + (size_t)slot * p.table_stride;

    // the queries of up to 16 heads: [rank from q1 | dr from q2], zero rows beyond the heads there are
    const int q_chunks = dk / 8;
    for (int e = tid; e < 16 * q_chunks; e += THREADS) {
        const int r = e / q_chunks, c = (e % q_chunks) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < heads_here) {
            const int h = h0 + r;
            v = c < p.rank ? *reinterpret_cast<const uint4*>(p.q1 + ((size_t)h * p.n_tokens + t) * p.rank + c)
                           : *reinterpret_cast<const uint4*>(p.q2 + ((size_t)t * p.heads + h) * p.dr + (c - p.rank));
        }
        *reinterpret_cast<uint4*>(qs + r * ld + c) = v;
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
    const int col0 = warp * NT * 8;                          // this warp's columns of the latent

    // Four threads bring one key's record: one look at the block table a thread and tile, 16-byte asynchronous copies
    // that land while the tile before is multiplied.
    auto fetch = [&](int tile, int buffer) {
        const int r = tid >> 2, j = first + tile * KEYS + r;
        const int row = j <= pos ? cache_row_of(table, j, p.page_size, -1, p.num_pages, p.error_flag) : -1;
        if ((tid & 3) == 0) key_rows_all[buffer * KEYS + r] = row;
        __nv_bfloat16* dst = ks_all + ((size_t)buffer * KEYS + r) * ld;
        for (int c = (tid & 3) * 8; c < dk; c += 32) {
            if (row >= 0) {
                const __nv_bfloat16* src = c < p.rank ? p.latent_pages + (size_t)row * p.rank + c
                                                      : p.part_pages + (size_t)row * p.dr + (c - p.rank);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst + c)), "l"(src) : "memory");
            } else {
                *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (tile_lo < tile_hi) fetch(tile_lo, 0);

    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int buffer = (tile - tile_lo) & 1;
        const __nv_bfloat16* ks = ks_all + (size_t)buffer * KEYS * ld;
        const int* key_rows = key_rows_all + buffer * KEYS;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                     // this tile is there (at first: the queries too); the one before is used up
        if (tile + 1 < tile_hi) fetch(tile + 1, buffer ^ 1);
        // ---- scores of keys 8 warp .. 8 warp + 7 for the 16 rows ----
        // four accumulators in turn: a product waits for the one before it only every fourth time
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const uint32_t a_base = smem_addr(qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8);
            const uint32_t b_base = smem_addr(ks + (warp * 8 + (lane & 7)) * ld + (lane >> 3) * 8);
            for (int k0 = 0; k0 < dk; k0 += 64) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                ldmatrix_x4(b_base + k0 * 2, b0, b1, b2, b3);               // k0..7, 8..15, 16..23, 24..31 of the 8 keys
                ldmatrix_x4(a_base + k0 * 2, a0, a1, a2, a3);
                mma_bf16(s0, a0, a1, a2, a3, b0, b1);
                if (k0 + 16 < dk) {
                    ldmatrix_x4(a_base + (k0 + 16) * 2, a0, a1, a2, a3);
                    mma_bf16(s1, a0, a1, a2, a3, b2, b3);
                }
                if (k0 + 32 < dk) {
                    ldmatrix_x4(b_base + (k0 + 32) * 2, b0, b1, b2, b3);
                    ldmatrix_x4(a_base + (k0 + 32) * 2, a0, a1, a2, a3);
                    mma_bf16(s2, a0, a1, a2, a3, b0, b1);
                    if (k0 + 48 < dk) {
                        ldmatrix_x4(a_base + (k0 + 48) * 2, a0, a1, a2, a3);
                        mma_bf16(s3, a0, a1, a2, a3, b2, b3);
                    }
                }
            }
        }
        float s[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] = (s0[e] + s1[e]) + (s2[e] + s3[e]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = g + (e >> 1) * 8, c = warp * 8 + tq * 2 + (e & 1);
            ss[r * (KEYS + 1) + c] = key_rows[c] >= 0 ? s[e] * p.scale_log2 : -INFINITY;
        }
        __syncthreads();
        // ---- softmax of rows g and g + 8 (every warp for itself), probabilities as the second product's A operand ----
        uint32_t pa[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float* srow = ss + (g + i * 8) * (KEYS + 1);
            float v[8];
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                v[kk * 4 + 0] = srow[kk * 16 + tq * 2];
                v[kk * 4 + 1] = srow[kk * 16 + tq * 2 + 1];
                v[kk * 4 + 2] = srow[kk * 16 + tq * 2 + 8];
                v[kk * 4 + 3] = srow[kk * 16 + tq * 2 + 9];
            }
            float top = v[0];
#pragma unroll
            for (int e = 1; e < 8; ++e) top = fmaxf(top, v[e]);
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
            top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
            const float new_max = fmaxf(row_max[i], top);
            const float safe = new_max == -INFINITY ? 0.f : new_max;
            const float correction = exp2f(row_max[i] - safe);              // 0 at the first tile with a key
            row_max[i] = new_max;
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[e] = exp2f(v[e] - safe);
                sum += v[e];
            }
            row_sum[i] = row_sum[i] * correction + sum;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                o[j][i * 2] *= correction;
                o[j][i * 2 + 1] *= correction;
            }
            // A fragment of k-step kk: (row g, keys 2t, 2t+1), (row g+8, ..), (row g, keys 2t+8, 2t+9), (row g+8, ..)
            pa[0][i] = pack2(v[0], v[1]);
            pa[0][i + 2] = pack2(v[2], v[3]);
            pa[1][i] = pack2(v[4], v[5]);
            pa[1][i + 2] = pack2(v[6], v[7]);
        }
        // ---- out += P latent, this warp's columns ----
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const int m = lane >> 3;
            const uint32_t v_base = smem_addr(ks + (kk * 16 + (m & 1) * 8 + (lane & 7)) * ld + col0 + (m >> 1) * 8);
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(v_base + j * 8 * 2, b0, b1, b2, b3);
                mma_bf16(o[j], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                if (j + 1 < NT) mma_bf16(o[j + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        row_sum[i] += __shfl_xor_sync(0xffffffffu, row_sum[i], 1);
        row_sum[i] += __shfl_xor_sync(0xffffffffu, row_sum[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + i * 8;
        if (r >= heads_here) continue;
        const size_t plane = (size_t)(h0 + r) * p.n_tokens + t;
        if (p.splits <= 1) {
            const float inv = row_sum[i] > 0.f ? 1.0f / row_sum[i] : 0.f;
            __nv_bfloat16* dst = p.out + plane * p.rank + col0 + tq * 2;
#pragma unroll
            for (int j = 0; j < NT; ++j) *reinterpret_cast<uint32_t*>(dst + j * 8) = pack2(o[j][i * 2] * inv, o[j][i * 2 + 1] * inv);
        } else {
            const size_t planes = (size_t)p.heads * p.n_tokens;
            float* dst = p.partial + ((size_t)blockIdx.z * planes + plane) * p.rank + col0 + tq * 2;
#pragma unroll
            for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][i * 2], o[j][i * 2 + 1]);
            if (warp == 0 && tq == 0) {
                float* ms = p.partial + (size_t)p.splits * planes * p.rank + ((size_t)blockIdx.z * planes + plane) * 2;
                ms[0] = row_max[i];
                ms[1] = row_sum[i];
            }
        }
    }
}

// out[h, t] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over the ranges that saw a key, in ascending order.
__global__ void latent_merge_kernel(LatentParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    if (p.slots[t] < 0) return;
    const size_t planes = (size_t)p.heads * p.n_tokens, plane = (size_t)h * p.n_tokens + t;
    const float* ms = p.partial + (size_t)p.splits * planes * p.rank;
    float top = -INFINITY;
    for (int s = 0; s < p.splits; ++s) top = fmaxf(top, ms[((size_t)s * planes + plane) * 2]);
    float total = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float m = ms[((size_t)s * planes + plane) * 2];
        if (m > -INFINITY) total += exp2f(m - top) * ms[((size_t)s * planes + plane) * 2 + 1];
    }
    const float inv = total > 0.f ? 1.0f / total : 0.f;
    for (int c = threadIdx.x; c < p.rank; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            const float m = ms[((size_t)s * planes + plane) * 2];
            if (m > -INFINITY) acc += exp2f(m - top) * p.partial[((size_t)s * planes + plane) * p.rank + c];
        }
        p.out[plane * p.rank + c] = __float2bfloat16_rn(acc * inv);
    }
}

size_t latent_smem_bytes(int rank, int dr) {
    const size_t ld = (size_t)rank + dr + PAD;
    return (16 + 2 * KEYS) * ld * 2 + 16 * (KEYS + 1) * sizeof(float) + 2 * KEYS * sizeof(int);
}

template <int NT>
int launch_latent(const LatentParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    static int configured = 0;             // the largest shared memory asked for so far
    if ((int)smem > configured) {
        if (cudaFuncSetAttribute(latent_attention_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return LIA_ERR_LAUNCH;
        }
        configured = (int)smem;
    }
    return lia_launch(latent_attention_kernel<NT>, grid, dim3(THREADS), smem, stream, p);
}
}  // namespace

// 1 if the kernel takes these sizes.
LIA_EXPORT int lia_latent_attention_accepts(int rank, int dr) {
    return rank > 0 && rank % 32 == 0 && rank <= 512 && dr > 0 && dr % 16 == 0 && dr <= 128 ? 1 : 0;
}

// Words of 32-bit scratch that `splits` ranges need.
LIA_EXPORT long long lia_latent_attention_partial_floats(int n_tokens, int heads, int rank, int splits) {
    return splits > 1 ? (long long)splits * heads * n_tokens * (rank + 2) : 0;
}

LIA_EXPORT int lia_latent_attention(const void* q1, const void* q2, const void* latent_pages, const void* part_pages,
                                    const int* positions, const int* slots, const int* block_table, int table_stride,
                                    void* out, float* partial, int n_tokens, int heads, int rank, int dr, int page_size,
                                    int window, float scale, int num_pages, int splits, int* error_flag,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return LIA_OK;
    if (!lia_latent_attention_accepts(rank, dr) || heads <= 0 || page_size <= 0 || splits < 1 || splits > 64 ||
        (splits > 1 && !partial))
        return LIA_ERR_SIZE;
    if (((uintptr_t)q1 & 15u) || ((uintptr_t)q2 & 15u) || ((uintptr_t)latent_pages & 15u) || ((uintptr_t)part_pages & 15u) ||
        ((uintptr_t)out & 3u) || ((uintptr_t)partial & 7u))
        return LIA_ERR_ALIGN;
    LatentParams p;
    p.q1 = (const __nv_bfloat16*)q1; p.q2 = (const __nv_bfloat16*)q2;
    p.latent_pages = (const __nv_bfloat16*)latent_pages; p.part_pages = (const __nv_bfloat16*)part_pages;
    p.positions = positions; p.slots = slots; p.block_table = block_table; p.out = (__nv_bfloat16*)out; p.partial = partial;
    p.n_tokens = n_tokens; p.heads = heads; p.rank = rank; p.dr = dr; p.table_stride = table_stride; p.page_size = page_size;
    p.window = window; p.num_pages = num_pages; p.splits = splits; p.scale_log2 = scale * LOG2E; p.error_flag = error_flag;
    const dim3 grid(n_tokens, (heads + 15) / 16, splits);
    if (grid.y > 65535) return LIA_ERR_SIZE;
    const size_t smem = latent_smem_bytes(rank, dr);
    int rc;
    switch (rank / 32) {
#define LIA_LATENT(NT) case NT: rc = launch_latent<NT>(p, grid, smem, stream); break;
        LIA_LATENT(1) LIA_LATENT(2) LIA_LATENT(3) LIA_LATENT(4) LIA_LATENT(5) LIA_LATENT(6) LIA_LATENT(7) LIA_LATENT(8)
        LIA_LATENT(9) LIA_LATENT(10) LIA_LATENT(11) LIA_LATENT(12) LIA_LATENT(13) LIA_LATENT(14) LIA_LATENT(15) LIA_LATENT(16)
#undef LIA_LATENT
        default: return LIA_ERR_SIZE;
    }
    if (rc != LIA_OK || splits <= 1) return rc;
    return lia_launch(latent_merge_kernel, dim3(n_tokens, heads), dim3(128), 0, stream, p);
}
