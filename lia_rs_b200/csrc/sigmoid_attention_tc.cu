// Attention with sigmoid weights (no softmax, no normalisation; see sigmoid_attention.cu for the definition) over the
// paged bfloat16 cache on the 5th-generation tensor cores, for prompt portions and single decoded tokens alike.
//
// A CTA owns up to 128 query rows = floor(128 / g) consecutive tokens x the g query heads of one kv head (a single decoded token
// is a portion of one token), and walks the keys its rows can see, 128 at a time, from the first key that the
// CTA's first token sees (the start of its block of `chunk` positions, or of its window) to its last token:
//     S = Q K^T      tcgen05.mma, M 128 (rows), N 128 (keys), K head_dim, accumulator in TMEM (two buffers)
//     weights        two threads per row, each with 64 of its 128 scores from tcgen05.ld:
//                    w = 1 / (1 + 2^(-(s scale + bias) log2 e)) in 32-bit, 0 for a key the row does not see; each
//                    weight is split into two bfloat16 numbers, hi = bf16(w) and lo = bf16(w - hi), which together
//                    hold 16 bits of it, and both go back to TMEM INTO THE SCORES' OWN BUFFER (hi in its columns
//                    0..63, lo in 64..127; the two threads of a row meet at a barrier between their loads and stores)
//     O += hi V + lo V   tcgen05.mma with the first operand from TMEM, M 128, N head_dim, K 128 keys, twice; V taken
//                    as it lies in its pages (an MN-major operand); accumulator in TMEM for the whole walk
// and at the end out = O * sigmoid(gate logit of the row's token and head).  There is no running maximum, no
// rescaling and no sum: the roles meet at fewer barriers than in the softmax kernel (attention_prefill_tc.cu), whose
// roles, loaders and tile layout this kernel shares.  MMAs of one thread run in the order they were issued, so the
// first product of tile j + 2, which overwrites the buffer that held the weights of tile j, needs no barrier
// against the second product of tile j.  Every wait on an mbarrier is bounded.
// What bounds a tile: two special-function instructions a weight (ex2, rcp): 32,768 per tile = 2,048 cycles of that
// pipe, against 512 + 1,024 cycles of MMA at head size 128.
//
// Head sizes: multiples of 8 up to 128, keys and values each their own; in shared memory the rows of Q, K and V are
// padded with zeros to D = 64 or 128 elements (what the swizzled tile and the MMA's K steps want), which costs the
// padding's share of the tensor work and nothing else.  Any g up to 128 (rows beyond (128 / g) g stay idle).  The caller uses the kernel for every size
// (sigmoid_attention.cu) for everything else.
#include "attention_tmem.cuh"

using namespace tc5;

namespace {
constexpr int ROWS = 128;                // query rows per CTA: the MMA's M
constexpr int KT = 128;                  // keys per tile: N of the first product, K of the second
constexpr int WEIGHT_WARPS = 8, LOAD_WARPS = 4;
constexpr int THREADS = (WEIGHT_WARPS + 1 + LOAD_WARPS) * 32;
constexpr int LOADERS = LOAD_WARPS * 32;
constexpr int STAGES = 3;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
    const __nv_bfloat16* q;          // [tokens, nq, d]
    const __nv_bfloat16* k_pages;    // [pages, page_size, nkv, d]
    const __nv_bfloat16* v_pages;    // [pages, page_size, nkv, dv]
    const int* segments;             // [n_segments][3]: first token's batch index, its position, count (portions of several tokens)
    const int* single_rows;          // [n_single]: batch indices of the single tokens
    const int* positions;            // [tokens]
    const int* slots;                // [tokens]
    const int* block_table;          // [slots, table_stride]
    const float* head_bias;          // [nq] or null
    const float* gate;               // logits: token t, head h at gate[t * gate_stride + h]; or null
    __nv_bfloat16* out;              // [tokens, nq, dv]
    int n_segments, portion_tiles, n_single, gate_stride, table_stride, nq, nkv, page_size, page_shift, window, chunk, tokens_per_tile;
    int d, dv;                       // the heads' real sizes (multiples of 8, at most D): rows are padded with zeros to D in shared memory
    float scale;
    int num_pages;
    int* error_flag;
    // A step of single tokens may leave the position encoding and the append to this kernel: `fused_rows` (32-bit, a row
    // of `fused_stride` floats a token: nq heads of d queries, nkv heads of d keys, nkv heads of dv values, as the
    // product before left them) replaces q; each CTA encodes its token's queries and key (rotary over adjacent pairs of
    // the first rotary_dim elements, frequencies `freq`, sine and cosine times `magnitude`), puts them into its tiles
    // and, with `write_kv`, the key and value into their page.
    // With `splits` > 1 (steps without portions) the tiles of every token's keys are cut into that many ranges (grid z), each
    // a CTA of its own that leaves its sum in `partial` ([splits][tokens * nq][dv] 32-bit); sigmoid_attention_sum_kernel
    // adds a row's ranges in ascending order and applies the gate.  There is nothing to renormalise: the ranges just add.
    int splits;
    float* partial;
    long long rows_total;            // tokens * nq
    const float* fused_rows;
    const float* freq;
    int fused_stride, rotary_dim, write_kv;
    float magnitude;
};

// Eight consecutive elements (from e0, a multiple of 8) of a head's 32-bit row, rotary-encoded where they lie within
// rotary_dim, as four bfloat16 pairs.  The arithmetic is that of rotary_pairs.cu.
__device__ __forceinline__ uint4 encoded_piece(const float* head, int e0, int pos, const float* freq, int rotary_dim, float magnitude) {
    const float4 lo = *reinterpret_cast<const float4*>(head + e0), hi = *reinterpret_cast<const float4*>(head + e0 + 4);
    float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = e0 + 2 * i;
        if (e < rotary_dim) {
            float sn, cs;
            sincosf((float)pos * freq[e >> 1], &sn, &cs);
            cs *= magnitude;
            sn *= magnitude;
            const float a = v[2 * i], b = v[2 * i + 1];
            v[2 * i] = a * cs - b * sn;
            v[2 * i + 1] = b * cs + a * sn;
        }
    }
    uint4 out;
    __nv_bfloat162 pair = __floats2bfloat162_rn(v[0], v[1]);
    out.x = *reinterpret_cast<uint32_t*>(&pair);
    pair = __floats2bfloat162_rn(v[2], v[3]);
    out.y = *reinterpret_cast<uint32_t*>(&pair);
    pair = __floats2bfloat162_rn(v[4], v[5]);
    out.z = *reinterpret_cast<uint32_t*>(&pair);
    pair = __floats2bfloat162_rn(v[6], v[7]);
    out.w = *reinterpret_cast<uint32_t*>(&pair);
    return out;
}
__device__ __forceinline__ void store_shared_16(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) first = max(first, (pos / chunk) * chunk);
    return first;
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
sigmoid_attention_tc_kernel(Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full[STAGES], v_full[STAGES], k_empty[STAGES], v_empty[STAGES], s_full[2], p_ready, o_done;
    __shared__ uint32_t tmem_base_slot;
    constexpr int PIECES = D / 8;                      // 16-byte pieces per row
    constexpr uint32_t Q_BYTES = ROWS * D * 2, KV_BYTES = KT * D * 2;
    constexpr int TMEM_COLS = 512;                     // two buffers of 128 columns (scores, then weights) and the output's D
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = smem_base, kv_s = q_s + Q_BYTES;   // kv_s: [stage][K, V]

    // ---- which tokens, which kv head: the tiles of the portions first (later tiles first: they have the most keys),
    //      then one CTA per single token ----
    const int group = p.nq / p.nkv;
    const int kvh = blockIdx.y;
    int q_offset = 0, seg_start = 0, seg_count = 0, tok0 = 0;
    bool found = false;
    if ((int)blockIdx.x < p.portion_tiles) {
        int tile = p.portion_tiles - 1 - blockIdx.x;
        for (int seg = 0; seg < p.n_segments; ++seg) {
            q_offset = p.segments[seg * 3];
            seg_start = p.segments[seg * 3 + 1];
            seg_count = p.segments[seg * 3 + 2];
            const int tiles = (seg_count + p.tokens_per_tile - 1) / p.tokens_per_tile;
            if (tile < tiles) { found = true; break; }
            tile -= tiles;
        }
        tok0 = tile * p.tokens_per_tile;
    } else if ((int)blockIdx.x - p.portion_tiles < p.n_single) {
        q_offset = p.single_rows[blockIdx.x - p.portion_tiles];
        seg_start = p.positions[q_offset];
        seg_count = 1;
        found = true;
    }
    const bool active = found && p.slots[q_offset] >= 0;
    const int tok_count = active ? min(p.tokens_per_tile, seg_count - tok0) : 0;
    const int pos_first = seg_start + tok0, pos_last = pos_first + tok_count - 1;
    const int key_end = pos_last + 1;
    const int key_begin_all = first_visible(pos_first, p.window, p.chunk);
    const int first_of_last = first_visible(max(pos_last, 0), p.window, p.chunk);    // what the CTA's last token sees first
    int key_begin_of_cta = key_begin_all, n_tiles = active ? (key_end - key_begin_all + KT - 1) / KT : 0;
    if (p.splits > 1) {                             // this CTA's range of the tiles
        const int per = (n_tiles + p.splits - 1) / p.splits;
        const int first = min(n_tiles, (int)blockIdx.z * per);
        n_tiles = min(n_tiles, first + per) - first;
        key_begin_of_cta += first * KT;
    }
    const int key_begin = key_begin_of_cta;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), LOADERS);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(smem_u32(&k_full[i]), LOADERS);
            mbar_init(smem_u32(&v_full[i]), LOADERS);
            mbar_init(smem_u32(&k_empty[i]), 1);
            mbar_init(smem_u32(&v_empty[i]), 1);
        }
        mbar_init(smem_u32(&s_full[0]), 1);
        mbar_init(smem_u32(&s_full[1]), 1);
        mbar_init(smem_u32(&p_ready), WEIGHT_WARPS * 32);
        mbar_init(smem_u32(&o_done), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == WEIGHT_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_base_slot, tmem_o = tmem_base_slot + 2 * KT;     // buffer b at tmem_s + b * KT
    pdl_launch_dependents();
    pdl_wait();                                   // q and this step's keys come from the kernel ahead

    if (warp > WEIGHT_WARPS && n_tiles > 0) {
        // ---- loaders: Q once, then the K and V tiles, each thread whole 16-byte pieces ----
        const int lt = threadIdx.x - (WEIGHT_WARPS + 1) * 32;            // 0..127
        const int* table = p.block_table + (size_t)p.slots[q_offset] * p.table_stride;
        auto bring_q = [&](bool encode) {
            for (int id = lt; id < ROWS * PIECES; id += LOADERS) {
                const int r = id / PIECES, piece = id % PIECES;
                const int tok = r / group, head = r % group;
                const bool valid = tok < tok_count && piece * 8 < p.d;
                if (encode) {
                    // the token's queries from the product's 32-bit row, encoded here (rows beyond its heads are zeros)
                    uint4 piece_bits = make_uint4(0u, 0u, 0u, 0u);
                    if (valid)
                        piece_bits = encoded_piece(p.fused_rows + (size_t)q_offset * p.fused_stride + (size_t)(kvh * group + head) * p.d, piece * 8,
                                                   seg_start, p.freq, p.rotary_dim, p.magnitude);
                    store_shared_16(q_s + tile_offset<ROWS>(r, piece), piece_bits);
                    continue;
                }
                const size_t src = ((size_t)(q_offset + tok0 + (tok < tok_count ? tok : 0)) * p.nq + kvh * group + head) * p.d + (valid ? piece * 8 : 0);
                cp_async_16(q_s + tile_offset<ROWS>(r, piece), p.q + src, valid);
            }
        };
        if (!p.fused_rows) bring_q(false);         // (a fused step encodes its queries below, behind the first tile's copies)
        cp_async_commit();                        // (Q is awaited below, with the first tile's copies already on their way)
        bool ok = true;
        int own_row = -1, own_piece = 0;              // fused step: the page row of the token's own key, if this thread holds a piece of it
        uint32_t own_at = 0;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % STAGES;
            // the keys' stage is free as soon as the first product of three tiles ago has read it, the values' stage
            // only after the second
            if (j >= STAGES && !mbar_wait(smem_u32(&k_empty[st]), ((uint32_t)(j / STAGES) & 1u) ^ 1u)) { ok = false; break; }
            const uint32_t ks = kv_s + (uint32_t)st * 2 * KV_BYTES, vs = ks + KV_BYTES;
            const int key0 = key_begin + j * KT;
            // PIECES lanes share a key row (their 16-byte pieces make one coalesced request); lane j of them looks
            // up the row of pass j
            {
                constexpr int ROWS_PER_PASS = LOADERS / PIECES, PASSES = KT / ROWS_PER_PASS;
                static_assert(PASSES <= PIECES, "one lane per pass");
                const int sub = lt / PIECES, piece = lt % PIECES, lane_group = (lane / PIECES) * PIECES;
                int my_row = -1, rows[PASSES];
                int own = -1;                          // the pass whose row is the token's own key (encoded here, not read)
                if (piece < PASSES) {
                    const int key = key0 + sub + piece * ROWS_PER_PASS;
                    if (key < key_end) my_row = cache_row_of(table, key, p.page_size, p.page_shift, p.num_pages, p.error_flag);
                }
#pragma unroll
                for (int i = 0; i < PASSES; ++i) {
                    const int row = __shfl_sync(0xffffffffu, my_row, lane_group + i);
                    const bool mine = p.fused_rows && key0 + sub + i * ROWS_PER_PASS == pos_last;
                    if (mine) own = i;
                    const bool valid = row >= 0 && piece * 8 < p.d && !mine;
                    const size_t src = ((size_t)(row >= 0 ? row : 0) * p.nkv + kvh) * p.d + (valid ? piece * 8 : 0);
                    const uint32_t at = tile_offset<KT>(sub + i * ROWS_PER_PASS, piece);
                    cp_async_16(ks + at, p.k_pages + src, valid);
                    rows[i] = row;
                }
                cp_async_commit();
                if (j >= STAGES && !mbar_wait(smem_u32(&v_empty[st]), ((uint32_t)(j / STAGES) & 1u) ^ 1u)) { ok = false; break; }
#pragma unroll
                for (int i = 0; i < PASSES; ++i) {
                    const bool valid = rows[i] >= 0 && piece * 8 < p.dv && i != own;
                    const size_t src = ((size_t)(rows[i] >= 0 ? rows[i] : 0) * p.nkv + kvh) * p.dv + (valid ? piece * 8 : 0);
                    cp_async_16(vs + tile_offset<KT>(sub + i * ROWS_PER_PASS, piece), p.v_pages + src, valid);
                }
                cp_async_commit();
                own_row = -1;
#pragma unroll
                for (int i = 0; i < PASSES; ++i)
                    if (i == own) { own_row = rows[i]; own_at = tile_offset<KT>(sub + i * ROWS_PER_PASS, piece); }
                own_piece = piece;
            }
            if (j == 0) {
                if (p.fused_rows) bring_q(true);
                asm volatile("cp.async.wait_group 2;" ::: "memory");    // Q has landed (groups complete in the order they were made)
                fence_async_smem();
                mbar_arrive(smem_u32(&q_full));
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");        // the keys have landed
            const float* fused = p.fused_rows ? p.fused_rows + (size_t)q_offset * p.fused_stride : nullptr;
            if (own_row >= 0 && own_piece * 8 < p.d) {
                // the token's own key: encoded, into the tile (over the zeros its copy left) and into its page
                const uint4 bits = encoded_piece(fused + (size_t)(p.nq + kvh) * p.d, own_piece * 8, pos_last, p.freq, p.rotary_dim, p.magnitude);
                store_shared_16(ks + own_at, bits);
                if (p.write_kv) *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(p.k_pages) + ((size_t)own_row * p.nkv + kvh) * p.d + own_piece * 8) = bits;
            }
            fence_async_smem();
            mbar_arrive(smem_u32(&k_full[st]));
            cp_async_wait_all();
            if (own_row >= 0 && own_piece * 8 < p.dv) {
                const uint4 bits = encoded_piece(fused + (size_t)(p.nq + p.nkv) * p.d + (size_t)kvh * p.dv, own_piece * 8, pos_last, p.freq, 0, 1.0f);
                store_shared_16(vs + own_at, bits);
                if (p.write_kv) *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(p.v_pages) + ((size_t)own_row * p.nkv + kvh) * p.dv + own_piece * 8) = bits;
            }
            fence_async_smem();
            mbar_arrive(smem_u32(&v_full[st]));
        }
        if (!ok && p.error_flag) atomicExch(p.error_flag, 3);
    } else if (warp == WEIGHT_WARPS && lane == 0 && n_tiles > 0) {
        // ---- MMA issuer ----
        const uint32_t idesc_s = instr_desc(ROWS, KT), idesc_o = instr_desc_b_mn(ROWS, D);
        bool ok = mbar_wait(smem_u32(&q_full), 0u);
        static_assert(ROWS == KT, "Q and K tiles share their offsets");
        const uint64_t desc_q0 = smem_desc(q_s), desc_kv0 = smem_desc(kv_s), desc_v0 = smem_desc_mn(kv_s + KV_BYTES, KT * 128, 1024);
        // S_j = Q K_j^T into buffer j & 1, issued one tile ahead of the second product of the tile before.  The
        // buffer held the weights of tile j - 2, whose second product was issued earlier by this thread.
        auto first_product = [&](int j) {
            const int st = j % STAGES;
            if (!mbar_wait(smem_u32(&k_full[st]), (uint32_t)(j / STAGES) & 1u)) { ok = false; return; }
            tc_fence_after();
            const uint64_t desc_k = desc_kv0 + (uint64_t)((uint32_t)st * (2 * KV_BYTES >> 4));
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t offset = (uint64_t)(((kk >> 2) * (ROWS * 128) + (kk & 3) * 32) >> 4);
                tc_mma(tmem_s + (uint32_t)((j & 1) * KT), desc_q0 + offset, desc_k + offset, idesc_s, kk > 0 ? 1u : 0u);
            }
            tc_commit(smem_u32(&s_full[j & 1]));
            tc_commit(smem_u32(&k_empty[st]));
        };
        if (ok) first_product(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % STAGES;
            const uint64_t desc_v = desc_v0 + (uint64_t)((uint32_t)st * (2 * KV_BYTES >> 4));
            if (j + 1 < n_tiles) first_product(j + 1);
            if (!ok) break;
            if (!mbar_wait(smem_u32(&v_full[st]), (uint32_t)(j / STAGES) & 1u)) { ok = false; break; }
            if (!mbar_wait(smem_u32(&p_ready), (uint32_t)j & 1u)) { ok = false; break; }
            tc_fence_after();
            const uint32_t weights = tmem_s + (uint32_t)((j & 1) * KT);          // hi at column 0, lo at column 64
#pragma unroll
            for (int part = 0; part < 2; ++part) {
#pragma unroll
                for (int ks16 = 0; ks16 < KT / 16; ++ks16)
                    tc_mma_ts(tmem_o, weights + (uint32_t)(part * (KT / 2) + ks16 * 8), desc_v + (uint64_t)(ks16 * (2048 >> 4)), idesc_o,
                              (j > 0 || ks16 > 0 || part > 0) ? 1u : 0u);
            }
            tc_commit(smem_u32(&v_empty[st]));
            if (j == n_tiles - 1) tc_commit(smem_u32(&o_done));
        }
        if (!ok && p.error_flag) atomicExch(p.error_flag, 3);
    } else if (warp < WEIGHT_WARPS && n_tiles > 0) {
        // ---- weights: warp w and warp w + 4 share the rows of TMEM lanes 32 (w % 4) ..; each takes half the keys of
        //      a tile and half the output's columns ----
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;                                  // 0..127
        const int tok = r / group, head = r % group;
        const bool row_ok = tok < tok_count;
        const int pos = row_ok ? pos_first + tok : -1;                      // a row beyond the portion sees nothing and is never written
        const int row_first = row_ok ? first_visible(pos, p.window, p.chunk) : 0;
        const uint32_t lane_base = ((uint32_t)(quarter * 32) << 16);
        constexpr int HALF = KT / 2;
        const float bias = p.head_bias ? p.head_bias[kvh * group + head] : 0.f;
        const float a = -p.scale * LOG2E, b = -bias * LOG2E;                // w = 1 / (1 + 2^(a s + b))
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int tile_first = key_begin + j * KT;
            const int key0 = tile_first + half * HALF;                      // this thread's first key of the tile
            if (!mbar_wait(smem_u32(&s_full[j & 1]), ((uint32_t)j >> 1) & 1u)) { ok = false; break; }
            tc_fence_after();
            // every row sees every key of the tile unless the tile reaches past the CTA's first token or begins before
            // what its last token sees first; rows beyond the portion are never written
            const bool masked = tile_first + KT - 1 > pos_first || tile_first < first_of_last;
            uint32_t raw[HALF];
            tmem_load64_nowait(tmem_s + (uint32_t)((j & 1) * KT + half * HALF) + lane_base, raw);
            tmem_load_wait();
            tc_fence_before();
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");        // the row's other thread has its scores too
            tc_fence_after();
            uint32_t low[HALF / 2];
#pragma unroll
            for (int c = 0; c < HALF; c += 2) {
                float w0 = rcp_approx(1.0f + ex2_approx(fmaf(__uint_as_float(raw[c]), a, b)));
                float w1 = rcp_approx(1.0f + ex2_approx(fmaf(__uint_as_float(raw[c + 1]), a, b)));
                if (masked) {
                    const int key = key0 + c;
                    if (key < row_first || key > pos) w0 = 0.f;
                    if (key + 1 < row_first || key + 1 > pos) w1 = 0.f;
                }
                const __nv_bfloat162 hi = __floats2bfloat162_rn(w0, w1);
                const uint32_t hi_bits = *reinterpret_cast<const uint32_t*>(&hi);
                const __nv_bfloat162 lo = __floats2bfloat162_rn(w0 - __uint_as_float(hi_bits << 16), w1 - __uint_as_float(hi_bits & 0xffff0000u));
                raw[c >> 1] = hi_bits;
                low[c >> 1] = *reinterpret_cast<const uint32_t*>(&lo);
            }
            const uint32_t buffer = tmem_s + lane_base + (uint32_t)((j & 1) * KT);
            tmem_store32(buffer + (uint32_t)(half * (HALF / 2)), raw);
            tmem_store32(buffer + (uint32_t)(KT / 2 + half * (HALF / 2)), low);
            tmem_store_wait();
            tc_fence_before();
            mbar_arrive(smem_u32(&p_ready));
        }
        // ---- the row's output times its gate: each of the row's two threads writes half the columns ----
        if (ok && !mbar_wait(smem_u32(&o_done), 0u)) ok = false;
        tc_fence_after();
        if (ok && p.splits > 1) {
            // this range's share of the row, as it stands
            const int t = q_offset + tok0 + (row_ok ? tok : 0);
            float* dst = p.partial + ((size_t)blockIdx.z * p.rows_total + (size_t)t * p.nq + kvh * group + head) * p.dv;
#pragma unroll 1
            for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 16) {
                float o[16];
                tmem_load16(tmem_o + lane_base + (uint32_t)c0, o);
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 16; c += 4)
                        if (c0 + c < p.dv) *reinterpret_cast<float4*>(dst + c0 + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
                }
            }
        } else if (ok) {
            const int t = q_offset + tok0 + (row_ok ? tok : 0);
            float g = 1.0f;
            if (p.gate && row_ok) g = 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.gate_stride + kvh * group + head]));
            __nv_bfloat16* dst = p.out + ((size_t)t * p.nq + kvh * group + head) * p.dv;
#pragma unroll 1
            for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 16) {
                float o[16];
                tmem_load16(tmem_o + lane_base + (uint32_t)c0, o);           // every lane takes part in the load
                if (row_ok) {
                    uint32_t packed[8];
#pragma unroll
                    for (int c = 0; c < 16; c += 2) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(o[c] * g, o[c + 1] * g);
                        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    if (c0 < p.dv) *reinterpret_cast<uint4*>(dst + c0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    if (c0 + 8 < p.dv) *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        } else if (lane == 0 && p.error_flag) {
            atomicExch(p.error_flag, 3);
        }
    }
    if (n_tiles == 0 && p.splits > 1 && active && threadIdx.x < ROWS) {
        // a range without tiles (fewer tiles than ranges): its share is nothing
        const int r = threadIdx.x, tok = r / group, head = r % group;
        if (tok < tok_count) {
            float* dst = p.partial + ((size_t)blockIdx.z * p.rows_total + (size_t)(q_offset + tok0 + tok) * p.nq + kvh * group + head) * p.dv;
            for (int c = 0; c < p.dv; ++c) dst[c] = 0.f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == WEIGHT_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_slot), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// out[t, h, :] = sigmoid(gate[t, h]) * sum over the ranges, in ascending order, of their shares: a CTA per single token,
// a thread per (head, 4 elements).
__global__ void sigmoid_attention_sum_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = p.single_rows[blockIdx.x];
    if (t < 0 || p.slots[t] < 0) return;
    const int quads = p.dv / 4;
    for (int item = threadIdx.x; item < p.nq * quads; item += blockDim.x) {
        const int h = item / quads, c = (item % quads) * 4;
        const size_t at = ((size_t)t * p.nq + h) * p.dv + c;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < p.splits; ++z) {
            const float4 part = *reinterpret_cast<const float4*>(p.partial + (size_t)z * p.rows_total * p.dv + at);
            sum.x += part.x; sum.y += part.y; sum.z += part.z; sum.w += part.w;
        }
        const float g = p.gate ? 1.0f / (1.0f + expf(-p.gate[(size_t)t * p.gate_stride + h])) : 1.0f;
        const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * g, sum.y * g), hi = __floats2bfloat162_rn(sum.z * g, sum.w * g);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.out + at) = packed;
    }
}

template <int D>
int launch(const Params& p, cudaStream_t stream) {
    const size_t smem = (size_t)ROWS * D * 2 + (size_t)STAGES * 2 * KT * D * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(sigmoid_attention_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return LIA_ERR_LAUNCH;
        configured = true;
    }
    const int rc = lia_launch(sigmoid_attention_tc_kernel<D>, dim3(p.portion_tiles + p.n_single, p.nkv, p.splits), dim3(THREADS), smem, stream, p);
    if (rc != LIA_OK || p.splits <= 1) return rc;
    return lia_launch(sigmoid_attention_sum_kernel, dim3(p.n_single), dim3(256), 0, stream, p);
}
}  // namespace

// Tokens of a portion that one CTA takes for `group` query heads per kv head, key head size d and value head size dv
// (0: this kernel does not take the combination; use lia_sigmoid_attention_generic).  Head sizes: multiples of 8 up to 128.
LIA_EXPORT int lia_sigmoid_attention_tc_tokens_per_tile(int group, int d, int dv) {
    if (d <= 0 || dv <= 0 || d % 8 || dv % 8 || d > 128 || dv > 128) return 0;
    return group >= 1 && group <= ROWS ? ROWS / group : 0;       // a group that does not divide 128 leaves the last rows idle
}

// q [tokens, nq, d], out [tokens, nq, dv] bfloat16; pages as lia_sigmoid_attention_generic (bfloat16).  `segments`
// ([n_segments][3] int32: first batch index, first position, count) lists the portions of several tokens and
// `portion_tiles` = sum over them of ceil(count / tokens_per_tile); `single_rows` lists the n_single batch indices of
// single tokens, whose positions come from `positions`.  head_bias, gate, gate_stride, window, chunk: as there.
// `fused_rows` (optional, only for a step without portions): see Params; q is then not read.  `splits` > 1 (only without
// portions): see Params; `partial` then holds splits * n_tokens * nq * dv 32-bit words, n_tokens the tokens that out covers.
LIA_EXPORT int lia_sigmoid_attention_tc(const void* q, const void* k_pages, const void* v_pages, const int* segments,
                                        int n_segments, int portion_tiles, const int* single_rows, int n_single,
                                        const int* positions, const int* slots, const int* block_table, int table_stride,
                                        void* out, int nq, int nkv, int d, int dv, int page_size, int window, int chunk,
                                        float scale, const float* head_bias, const float* gate, int gate_stride,
                                        int num_pages, const float* fused_rows, int fused_stride, const float* freq,
                                        int rotary_dim, float magnitude, int write_kv, int splits, float* partial, int n_tokens,
                                        int* error_flag, cudaStream_t stream) {
    if (portion_tiles + n_single <= 0) return LIA_OK;
    if (fused_rows && (portion_tiles > 0 || fused_stride < (nq + nkv) * d + nkv * dv || fused_stride % 4 || ((uintptr_t)fused_rows & 15u) ||
                       rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1) || (rotary_dim > 0 && !freq)))
        return LIA_ERR_SIZE;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || nkv > 65535 || portion_tiles < 0 || n_single < 0) return LIA_ERR_SIZE;
    if (splits < 1 || splits > 32 || (splits > 1 && (portion_tiles > 0 || !partial || n_tokens <= 0 || ((uintptr_t)partial & 15u)))) return LIA_ERR_SIZE;
    const int per_tile = lia_sigmoid_attention_tc_tokens_per_tile(nq / nkv, d, dv);
    if (per_tile == 0) return LIA_ERR_SIZE;
    if (((uintptr_t)q & 15u) || ((uintptr_t)out & 15u) || ((uintptr_t)k_pages & 15u) || ((uintptr_t)v_pages & 15u)) return LIA_ERR_ALIGN;
    Params p;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.segments = segments; p.single_rows = single_rows; p.positions = positions; p.slots = slots; p.block_table = block_table;
    p.head_bias = head_bias; p.gate = gate; p.out = (__nv_bfloat16*)out;
    p.n_segments = n_segments; p.portion_tiles = portion_tiles; p.n_single = n_single; p.gate_stride = gate_stride;
    p.table_stride = table_stride; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window; p.chunk = chunk;
    p.tokens_per_tile = per_tile; p.d = d; p.dv = dv; p.scale = scale; p.num_pages = num_pages; p.error_flag = error_flag;
    p.fused_rows = fused_rows; p.fused_stride = fused_stride; p.freq = freq; p.rotary_dim = rotary_dim; p.magnitude = magnitude;
    p.write_kv = write_kv;
    p.splits = splits; p.partial = partial; p.rows_total = (long long)n_tokens * nq;
    p.page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if (page_size == (1 << b)) p.page_shift = b;
    if (d > 64 || dv > 64) return launch<128>(p, stream);        // rows padded with zeros to 128 elements, or to 64
    return launch<64>(p, stream);
}
