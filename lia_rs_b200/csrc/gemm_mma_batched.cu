// Many products of one shape in one launch on the tensor cores (bfloat16, mma.sync):
//     out[b][m, n] = sum_k A[b][m, k] * W[b][n, k],   b < batch
// each with a matrix of its own and rows of its own, as the heads of an attention whose keys and values are expansions
// of a shared latent need them (a head's share of the expansion is a small matrix; all tokens pass through it).
//
// A CTA owns a 128 x 64 tile of one product: eight warps of 16 rows each, the whole tile's columns per warp (32
// accumulators a thread), K in steps of 32 through two shared-memory buffers filled by 16-byte asynchronous copies a step
// ahead, operands by `ldmatrix`.  Rows, columns and K beyond the product's sizes are zeros in shared memory.  The
// products here have short K (a head's size or a latent's rank), so a CTA lives for 4 to 16 steps: what matters is that
// all of them run at once and stream their operands from L2.
//
// K and the row strides multiples of 8 elements, 16-byte aligned bases and batch strides; N and the output's strides even.
#include "common.cuh"

namespace {
constexpr int BM = 128, BN = 64, BK = 32, LDS = BK + 8, THREADS = 256;

__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes of row `row` (if < rows) at element k (if < K) of a matrix with row stride ld into shared memory, else zeros
__device__ __forceinline__ void bring(__nv_bfloat16* dst, const __nv_bfloat16* base, int row, int rows, int k, int K, long long ld) {
    if (row < rows && k < K)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr(dst)), "l"(base + (size_t)row * ld + k) : "memory");
    else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
}

__global__ void __launch_bounds__(THREADS)
gemm_mma_batched_kernel(const __nv_bfloat16* __restrict__ A, long long lda, long long a_batch,
                        const __nv_bfloat16* __restrict__ W, long long ldw, long long w_batch,
                        __nv_bfloat16* __restrict__ out, long long ldo, long long out_batch, int M, int N, int K) {
    __shared__ __align__(16) __nv_bfloat16 as[2][BM][LDS];
    __shared__ __align__(16) __nv_bfloat16 ws[2][BN][LDS];
    pdl_launch_dependents();
    pdl_wait();
    A += (size_t)blockIdx.z * a_batch;
    W += (size_t)blockIdx.z * w_batch;
    out += (size_t)blockIdx.z * out_batch;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    auto fetch = [&](int k0, int buffer) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {                      // 128 rows x 4 pieces of 8 elements
            const int e = tid + i * THREADS, r = e >> 2, c = (e & 3) * 8;
            bring(&as[buffer][r][c], A, m0 + r, M, k0 + c, K, lda);
        }
        {
            const int r = tid >> 2, c = (tid & 3) * 8;     // 64 rows x 4 pieces
            bring(&ws[buffer][r][c], W, n0 + r, N, k0 + c, K, ldw);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int steps = (K + BK - 1) / BK;
    fetch(0, 0);
    for (int s = 0; s < steps; ++s) {
        const int buffer = s & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (s + 1 < steps) fetch((s + 1) * BK, buffer ^ 1);
        uint32_t a[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
            ldsm_x4(saddr(&as[buffer][warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk * 16 + (lane >> 4) * 8]), a[kk][0], a[kk][1],
                    a[kk][2], a[kk][3]);
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            uint32_t b0, b1, b2, b3;                        // k 0..7, 8..15, 16..23, 24..31 of columns 8j..8j+7
            ldsm_x4(saddr(&ws[buffer][j * 8 + (lane & 7)][(lane >> 3) * 8]), b0, b1, b2, b3);
            mma16816(acc[j], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
            mma16816(acc[j], a[1][0], a[1][1], a[1][2], a[1][3], b2, b3);
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + warp * 16 + g + i * 8;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            const int n = n0 + j * 8 + tq * 2;
            if (n < N) {                                     // N is even: n + 1 < N too
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[j][i * 2], acc[j][i * 2 + 1]);
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)m * ldo + n) = v;
            }
        }
    }
}
}  // namespace

// 1 if the kernel takes these sizes and strides (in elements) and these addresses.
LIA_EXPORT int lia_gemm_mma_batched_accepts(const void* A, long long lda, long long a_batch, const void* W, long long ldw,
                                            long long w_batch, const void* out, long long ldo, long long out_batch, int M,
                                            int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 || N % 2 || lda < K || ldw < K || ldo < N) return 0;
    if (lda % 8 || ldw % 8 || a_batch % 8 || w_batch % 8 || ldo % 2 || out_batch % 2) return 0;
    if (((uintptr_t)A & 15u) || ((uintptr_t)W & 15u) || ((uintptr_t)out & 3u)) return 0;
    return 1;
}

LIA_EXPORT int lia_gemm_mma_batched(const void* A, long long lda, long long a_batch, const void* W, long long ldw,
                                    long long w_batch, void* out, long long ldo, long long out_batch, int batch, int M,
                                    int N, int K, cudaStream_t stream) {
    if (batch <= 0 || M <= 0 || N <= 0) return LIA_OK;
    if (!lia_gemm_mma_batched_accepts(A, lda, a_batch, W, ldw, w_batch, out, ldo, out_batch, M, N, K)) return LIA_ERR_SIZE;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    if (grid.y > 65535 || batch > 65535) return LIA_ERR_SIZE;
    return lia_launch(gemm_mma_batched_kernel, grid, dim3(THREADS), 0, stream, (const __nv_bfloat16*)A, lda, a_batch,
                      (const __nv_bfloat16*)W, ldw, w_batch, (__nv_bfloat16*)out, ldo, out_batch, M, N, K);
}
