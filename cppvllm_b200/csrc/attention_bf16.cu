// Tensor-core attention over the paged cache for bf16, head sizes 64 and 128.
//
//   cvb_attn_prefill_bf16  prompt portions (requests with more than one token in the step): flash attention with a
//                          causal offset, reading ALL keys (earlier portions' and the step's own) from the pages.
//   cvb_attn_decode_bf16   single decoded tokens: the key range of every (request, kv head) is cut into `splits`
//                          chunks that run in parallel.  Up to 16 chunks are the blocks of one thread-block cluster and
//                          merge their partial (max, sum, output) triples through distributed shared memory; more go
//                          through scratch memory and cvb_attn_decode_merge (launched by the same entry point).
//   cvb_attn_decode_fused_bf16  the same from the projection's raw output: the kernel also norms and rotates the
//                          queries and the new key and writes the new key and value to the cache.
//
// Both kernels put the query heads that share a kv head next to each other in the M dimension of the matrix
// product (row r = token r / g, head kvh * g + r % g), so a key/value tile is loaded once for the whole group.
// Scores, softmax statistics and the output accumulator are float; probabilities are rounded to bf16 for the
// second product, as flash attention does.  Formulas as in attention_general.cu (reference
// kernels/paged_attention.cu:89-359: scale * q.k, keys lo..p, online softmax, o = sum p v / l).
//
// Key and value tiles are fetched by TMA (cp.async.bulk.tensor.2d through a tensor map of the page pool seen as
// rows of head_dim elements; one box per page and 64-column half, 128-byte swizzle, completion on an mbarrier
// with a transaction count), issued by a producer warp into a ring of stages: "full" barriers tell the four
// consumer warps that a tile has landed, "empty" barriers (one arrival per consumer warp) give the stage back.  A box whose keys lie outside
// the request's range is fetched from the nearest page inside it, so every tile brings the same number of
// bytes and never touches a page the request does not own; such keys are excluded by the mask.  Waits on the
// mbarrier are bounded: if one runs out, the block records error 5 and carries on to its end.  The query tile
// comes by cp.async.  The matrix products are mma.sync.m16n8k16 (bf16 in, float accumulate); ldmatrix reads the
// swizzled tiles without bank conflicts.
#include "sm100.cuh"
#include "tensor_map.cuh"
#include "attention_bf16.h"

namespace cvb {

constexpr int kBN = 64;                 // keys per tile
constexpr int kConsumers = 128;         // 4 warps that compute
constexpr int kThreads = kConsumers + 32; // plus one warp that issues the TMA copies
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// element offset of 16-byte chunk `c` of row `r` in the query tile (rows of HD bf16, chunks XOR-swizzled by row)
template <int HD> __device__ __forceinline__ int swz(int r, int c) { return r * HD + ((c ^ (r & 7)) << 3); }

// element offset of chunk `c` of key row `r` in a key/value tile as TMA lays it out: HD/64 halves of
// [64 rows][64 columns], each 128-byte row with its 16-byte chunks XOR-ed by (row & 7) (the 128-byte swizzle)
__device__ __forceinline__ int kv_off(int r, int c) { return ((c >> 3) << 12) + (r << 6) + (((c & 7) ^ (r & 7)) << 3); }

struct AttnParams {
    __nv_bfloat16* out;                 // [T, H, HD]
    const __nv_bfloat16* q;             // [T, H, HD]
    const int* block_tables;            // [S, table_width]
    const int* cu_seqlens;              // [S + 1]
    const int* positions;               // [T]
    int table_width, S, H, KV, page_size, window, num_pages;
    int box_rows;                       // rows of one TMA box: min(page_size, 64)
    float scale_log2;                   // scale * log2(e)
    int* err;
    // decode only
    float* part_o;                      // [S, KV, splits, 16, HD]
    float* part_ml;                     // [S, KV, splits, 16, 2]
    int splits;
    int cluster;                        // 1: the splits of a (request, kv head) are one thread-block cluster
    // decode with the projection's raw output (qkv != nullptr): queries are normed and rotated in the kernel, the new
    // key and value are written to the cache by the block whose keys include the token's own position
    const __nv_bfloat16* qkv;           // [T, H + 2 KV, HD]
    const float* q_w;                   // [HD] per-head norm weights, or nullptr for no norm
    const float* k_w;
    const float* cos_t;                 // [max_pos, HD / 2], or nullptr for no rotation
    const float* sin_t;
    const int* slots;                   // [T] cache slot (page * page_size + offset) of each token
    __nv_bfloat16* cache;               // the pages the tensor map describes
    int64_t cache_elems;
    int max_pos;
    float qk_eps;
};

// Issued by one WARP: fetch keys [key0, key0 + 64) of one kv head, K then V, into a stage.  `stage` points at the K
// tile; the V tile follows it.  Each lane issues one TMA box (a page or 64 keys, a 64-column half, K or V), so the
// block-table reads of a tile are in flight together.  Lane 0 waits for the stage to be free (`empty`, unless null) and
// arms the barrier before anyone copies.
template <int HD>
__device__ __forceinline__ void tma_issue_tile(__nv_bfloat16* stage, uint64_t* bar, uint64_t* empty, uint32_t empty_parity,
                                               const CUtensorMap* map, const AttnParams& p, const int* table, int kvh,
                                               int key0, int key_lo, int key_hi, int lane) {
    constexpr int kTileElems = kBN * HD;
    const int per_kv = (kBN / p.box_rows) * (HD / 64);            // boxes of K (and of V) in a tile: 1 to 8
    const int which = lane / per_kv;                              // 0: K, 1: V, above: idle lanes
    const int box = (lane % per_kv) / (HD / 64), half = lane % (HD / 64);
    int row = 0;
    if (which < 2) {
        int key = min(max(key0 + box * p.box_rows, key_lo), key_hi);   // outside the range: the nearest key inside it
        key -= key % p.box_rows;                                      // boxes start on multiples of their size
        const int slot = key / p.page_size;
        int page = slot < p.table_width ? table[slot] : -1;
        if (page < 0 || page >= p.num_pages) { atomicExch(p.err, 4); page = 0; }
        row = ((page * 2 + which) * p.KV + kvh) * p.page_size + key % p.page_size;
    }
    if (lane == 0) {
        if (empty != nullptr) mbar_wait(empty, empty_parity, p.err);
        mbar_expect_tx(bar, 2u * kTileElems * sizeof(__nv_bfloat16));
    }
    __syncwarp();
    if (which < 2) tma_load_2d(stage + which * kTileElems + half * 4096 + box * p.box_rows * 64, map, bar, half * 64, row);
}

// One warp: S[16 x NT*8] = Q[16 x HD] * K^T over NT/2 groups of 16 keys starting at tile row `krow0`.
template <int HD, int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const uint32_t (&qf)[HD / 16][4],
                                           const __nv_bfloat16* sK, int krow0, int lane) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            const int r = krow0 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int c = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b, sK + kv_off(r, c));
            mma_bf16(s[np * 2], qf[ks], b[0], b[1]);
            mma_bf16(s[np * 2 + 1], qf[ks], b[2], b[3]);
        }
    }
}

// One warp: O[16 x HD] += P[16 x NT*8] * V over the same keys.
template <int HD, int NT>
__device__ __forceinline__ void pv_product(float (&o)[HD / 8][4], const float (&s)[NT][4],
                                           const __nv_bfloat16* sV, int krow0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            uint32_t b[4];
            const int r = krow0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int c = dp * 2 + (lane >> 4);
            ldmatrix_x4_trans(b, sV + kv_off(r, c));
            mma_bf16(o[dp * 2], a, b[0], b[1]);
            mma_bf16(o[dp * 2 + 1], a, b[2], b[3]);
        }
    }
}

// Rows first_row .. last_row of a value tile in shared memory become zero (the lanes of one warp share the work).  Keys
// behind a request's last one lie in the same page of the cache as its last keys and come along with them; their
// probability is 0, but what a former holder of the page left there (an Inf, a NaN) times 0 would be NaN, so they must
// not meet the product as they are.  A warp clears the rows that it reads itself; warps that clear the same rows write
// the same zeros.
template <int HD>
__device__ __forceinline__ void clear_value_rows(__nv_bfloat16* sV, int first_row, int last_row, int lane) {
    constexpr int CPR = HD / 8;
    for (int i = lane; i < (last_row - first_row + 1) * CPR; i += 32)
        *reinterpret_cast<uint4*>(sV + kv_off(first_row + i / CPR, i % CPR)) = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();                                  // the next filling of the stage comes through the async proxy
    __syncwarp();
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Updates the running max and sum of the warp's two rows per thread, rescales the output accumulator and turns
// raw scores into probabilities p = 2^(s * scale_log2 - m).  Column n of the tile is key `key0 + n`; with MASK,
// keys outside [row_lo, row_hi] of their row are excluded (tiles that lie wholly inside every row's range skip
// the comparisons).
template <int HD, int NT, bool MASK>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[HD / 8][4], float (&m)[2], float (&l)[2],
                                             int key0, const int (&row_lo)[2], const int (&row_hi)[2],
                                             float scale_log2, int lane) {
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int half = e >> 1;
            if (MASK) {
                const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
                if (j < row_lo[half] || j > row_hi[half]) s[nt][e] = -INFINITY;
            }
            tile_max[half] = fmaxf(tile_max[half], s[nt][e]);
        }
    }
    float corr[2], m_scaled[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        tile_max[half] = fmaxf(tile_max[half], __shfl_xor_sync(0xffffffffu, tile_max[half], 1));
        tile_max[half] = fmaxf(tile_max[half], __shfl_xor_sync(0xffffffffu, tile_max[half], 2));
        const float m_new = fmaxf(m[half], tile_max[half] * scale_log2);      // scale > 0 keeps the order
        m_scaled[half] = m_new == -INFINITY ? 0.f : m_new;
        corr[half] = fast_exp2(m[half] - m_scaled[half]);                    // 2^(-inf) = 0 at the first tile
        m[half] = m_new;
    }
    float tile_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int half = e >> 1;
            const float pr = fast_exp2(fmaf(s[nt][e], scale_log2, -m_scaled[half]));   // excluded keys: 2^(-inf) = 0
            s[nt][e] = pr;
            tile_sum[half] += pr;
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) l[half] = l[half] * corr[half] + tile_sum[half];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }
}

// Carves the dynamic shared memory: stages (1024-byte aligned for the swizzle), then the query tile, then barriers.
template <int HD, int STAGES, int QROWS>
struct SmemPlan {
    static constexpr int kStageElems = 2 * kBN * HD;                      // K tile + V tile
    static constexpr size_t kBytes = 1024 + static_cast<size_t>(STAGES) * kStageElems * 2 + static_cast<size_t>(QROWS) * HD * 2 + 16 * STAGES;
    __nv_bfloat16* stages;
    __nv_bfloat16* q;
    uint64_t* bars;                      // [STAGES] full, then [STAGES] empty
    __device__ explicit SmemPlan(unsigned char* raw) {
        const uint32_t addr = smem_u32(raw);
        unsigned char* base = raw + ((1024u - (addr & 1023u)) & 1023u);
        stages = reinterpret_cast<__nv_bfloat16*>(base);
        q = stages + STAGES * kStageElems;
        bars = reinterpret_cast<uint64_t*>(q + QROWS * HD);
    }
};

// ---- prefill ---------------------------------------------------------------------------------------------------

constexpr int kPreStages = 2;

template <int HD>
__global__ void __launch_bounds__(kThreads)
attn_prefill_bf16_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnParams p, const int skip_single) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using Plan = SmemPlan<HD, kPreStages, 64>;
    Plan sm(smem_raw);
    constexpr int CPR = HD / 8;
    const int g = p.H / p.KV;
    const int tok_per_tile = 64 / g;
    const int kvh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // which request and which tile of it: walk the requests, counting tiles
    int seq = -1, q0 = 0, q_len = 0, cu0 = 0;
    {
        int tile = blockIdx.x;
        for (int s = 0; s < p.S; ++s) {
            const int a = p.cu_seqlens[s], n = p.cu_seqlens[s + 1] - a;
            if (skip_single && n == 1) continue;
            const int tiles = (n + tok_per_tile - 1) / tok_per_tile;
            if (tile < tiles) { seq = s; q0 = tile * tok_per_tile; q_len = n; cu0 = a; break; }
            tile -= tiles;
        }
    }
    if (seq < 0) return;
    const int n_tok = min(tok_per_tile, q_len - q0);
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int pos_first = p.positions[cu0 + q0];
    const int pos_last = p.positions[cu0 + q0 + n_tok - 1];
    const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int key_hi = pos_last;
    const int seq_last = p.positions[cu0 + q_len - 1];   // the request's last key in the cache after this step
    const int tile_begin = key_lo / kBN, n_tiles = key_hi / kBN - tile_begin + 1;

    uint64_t* full = sm.bars;
    uint64_t* empty = sm.bars + kPreStages;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kPreStages; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, kConsumers / 32); }
        mbar_fence_init();
    }
    // Q tile: row r = (token r / g, head kvh * g + r % g)
    for (int i = threadIdx.x; i < 64 * CPR; i += kThreads) {
        const int r = i / CPR, c = i % CPR;
        const int tok = r / g;
        const bool valid = tok < n_tok;
        const __nv_bfloat16* src = valid ? p.q + ((static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * HD + c * 8) : p.q;
        cp_async16(sm.q + swz<HD>(r, c), src, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();                                      // barriers are initialised, the query tile is in place

    if (warp == kConsumers / 32) {                        // ---- producer warp ----
        for (int it = 0; it < n_tiles; ++it) {
            const int st = it % kPreStages;
            tma_issue_tile<HD>(sm.stages + st * Plan::kStageElems, full + st, it >= kPreStages ? empty + st : nullptr,
                               ((it / kPreStages) - 1) & 1, &kv_map, p, table, kvh, (tile_begin + it) * kBN, key_lo, key_hi, lane);
        }
        return;
    }

    // ---- consumer warps: the two rows this thread owns in the warp's 16-row slab, and the warp's extremes ----
    int row_lo[2], row_hi[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = min(r / g, n_tok - 1);            // rows past the tile's tokens repeat the last one; never stored
        const int pos = p.positions[cu0 + q0 + tok];
        row_hi[half] = pos;
        row_lo[half] = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    }
    const bool warp_has_rows = warp * 16 < n_tok * g;
    const int warp_first_pos = p.positions[cu0 + q0 + min(n_tok - 1, (warp * 16) / g)];
    const int warp_last_pos = p.positions[cu0 + q0 + min(n_tok - 1, (warp * 16 + 15) / g)];
    const int warp_max_lo = p.window > 0 ? max(0, warp_last_pos - p.window + 1) : 0;

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], sm.q + swz<HD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it % kPreStages;
        const int key0 = (tile_begin + it) * kBN;
        // Every warp waits for the tile, also one that has nothing to add to it (its rows end before the tile:
        // causal): a warp may arrive on "empty" only once per filling of the stage, and the tile's arrival is
        // what tells it that the previous filling was given back by all four warps.
        mbar_wait(full + st, (it / kPreStages) & 1, p.err);
        if (warp_has_rows && key0 <= warp_last_pos) {
            const __nv_bfloat16* sK = sm.stages + st * Plan::kStageElems;
            __nv_bfloat16* sV = sm.stages + st * Plan::kStageElems + kBN * HD;
            if (key0 + kBN - 1 > seq_last) clear_value_rows<HD>(sV, max(0, seq_last + 1 - key0), kBN - 1, lane);
            float s[8][4];
            qk_product<HD, 8>(s, qf, sK, 0, lane);
            if (key0 + kBN - 1 <= warp_first_pos && key0 >= warp_max_lo)
                softmax_step<HD, 8, false>(s, o, m, l, key0, row_lo, row_hi, p.scale_log2, lane);
            else
                softmax_step<HD, 8, true>(s, o, m, l, key0, row_lo, row_hi, p.scale_log2, lane);
            pv_product<HD, 8>(o, s, sV, 0, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + st);
    }

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 1);
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = r / g;
        if (tok >= n_tok) continue;
        const float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * HD;
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[dt][half * 2] * inv, o[dt][half * 2 + 1] * inv);
        }
    }
}

// ---- decode ----------------------------------------------------------------------------------------------------

constexpr int kDecStages = 3;

template <int HD>
__global__ void __launch_bounds__(kThreads)
attn_decode_bf16_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnParams p) {
    // With the projection's raw output (the fused form) nothing that this kernel reads from the cache was written by
    // the kernels directly in front of it: the keys of earlier positions are older than this step, and the token's own
    // key and value are made here.  So the producer warp starts fetching keys at once, ahead of the dependency, and only
    // what reads the projection (and everything that writes) comes behind the wait.  Without the fused form the kernel in
    // front of this one has just written the new key into the cache: all of it waits.
    const bool fused = p.qkv != nullptr;
    if (!fused) pdl_wait();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using Plan = SmemPlan<HD, kDecStages, 16>;
    Plan sm(smem_raw);
    constexpr int CPR = HD / 8;
    const int g = p.H / p.KV;
    const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // with the projection's raw output every request brings exactly one token: token s belongs to request s
    const int cu0 = p.qkv != nullptr ? seq : p.cu_seqlens[seq];
    if (p.qkv == nullptr && p.cu_seqlens[seq + 1] - cu0 != 1) return;      // not a single decoded token
    const int pos = p.positions[cu0];
    const int key_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int key_hi = pos;
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int first_tile = key_lo / kBN, all_tiles = key_hi / kBN - first_tile + 1;
    const int per_split = (all_tiles + p.splits - 1) / p.splits;
    const int tile_begin = first_tile + split * per_split;
    const int n_tiles = max(0, min(first_tile + all_tiles, tile_begin + per_split) - tile_begin);

    float o[HD / 8][4];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (n_tiles > 0) {
        uint64_t* full = sm.bars;
        uint64_t* empty = sm.bars + kDecStages;
        __nv_bfloat16* newkv = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(sm.bars) + 64);   // [2][HD]
        const int tile_of_pos = pos / kBN;
        const bool owns_pos = p.qkv != nullptr && tile_of_pos >= tile_begin && tile_of_pos < tile_begin + n_tiles;
        if (warp == kConsumers / 32) {                                     // ---- producer warp ----
            // it sets up the barriers itself and starts fetching keys while the other warps prepare the queries
            if (lane == 0) {
                for (int i = 0; i < kDecStages; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, kConsumers / 32); }
                mbar_fence_init();
            }
            __syncwarp();
            asm volatile("bar.arrive 1, %0;\n" ::"n"(kThreads) : "memory");
            for (int it = 0; it < n_tiles; ++it) {
                const int st = it % kDecStages;
                tma_issue_tile<HD>(sm.stages + st * Plan::kStageElems, full + st, it >= kDecStages ? empty + st : nullptr,
                                   ((it / kDecStages) - 1) & 1, &kv_map, p, table, kvh, (tile_begin + it) * kBN, key_lo, key_hi, lane);
            }
        } else {                                                           // ---- consumer warps ----
            if (p.qkv == nullptr) {
                for (int i = threadIdx.x; i < 16 * CPR; i += kConsumers) {
                    const int r = i / CPR, c = i % CPR;
                    const bool valid = r < g;
                    const __nv_bfloat16* src = valid ? p.q + ((static_cast<int64_t>(cu0) * p.H + kvh * g + r) * HD + c * 8) : p.q;
                    cp_async16(sm.q + swz<HD>(r, c), src, valid);
                }
                cp_async_commit();
                cp_async_wait<0>();
            } else {
            pdl_wait();
            // Per-head norm and rotation of this kv head's queries, straight from the projection; CPR neighbouring lanes
            // own one head vector (16-byte chunks).  The block that owns the token's own position does the same for the
            // new key, copies the new value, and writes both to the cache and to shared memory.
            const int c = threadIdx.x % CPR, sub = threadIdx.x / CPR;
            constexpr int kPerPass = kConsumers / CPR;
            const bool first = c < CPR / 2;
            float cs[8], sn[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { cs[i] = 1.f; sn[i] = 0.f; }
            if (p.cos_t != nullptr) {
                int rp = pos;
                if (rp < 0 || rp >= p.max_pos) {
                    if (threadIdx.x == 0) atomicExch(p.err, 3);
                    rp = rp < 0 ? 0 : p.max_pos - 1;
                }
                const int e0 = (first ? c : c - CPR / 2) * 8;
                const float4* cr = reinterpret_cast<const float4*>(p.cos_t + static_cast<int64_t>(rp) * (HD / 2) + e0);
                const float4* sr = reinterpret_cast<const float4*>(p.sin_t + static_cast<int64_t>(rp) * (HD / 2) + e0);
                const float4 a0 = cr[0], a1 = cr[1], b0 = sr[0], b1 = sr[1];
                cs[0] = a0.x; cs[1] = a0.y; cs[2] = a0.z; cs[3] = a0.w; cs[4] = a1.x; cs[5] = a1.y; cs[6] = a1.z; cs[7] = a1.w;
                sn[0] = b0.x; sn[1] = b0.y; sn[2] = b0.z; sn[3] = b0.w; sn[4] = b1.x; sn[5] = b1.y; sn[6] = b1.z; sn[7] = b1.w;
                if (first) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) sn[i] = -sn[i];
                }
            }
            int64_t k_elem = -1;                                           // where the new key goes in the cache
            if (owns_pos) {
                const int slot = p.slots[cu0];
                if (slot >= 0) {
                    const int64_t page = slot / p.page_size, off = slot % p.page_size;
                    k_elem = (((page * 2) * p.KV + kvh) * p.page_size + off) * HD;
                    if (k_elem + static_cast<int64_t>(p.KV) * p.page_size * HD + HD > p.cache_elems) {
                        if (threadIdx.x == 0) atomicExch(p.err, 2);
                        k_elem = -1;
                    }
                }
            }
            const int n_tasks = g + (owns_pos ? 2 : 0);                    // g query heads, then the new key, then the value
            const int n_heads = p.H + 2 * p.KV;
            for (int t0 = 0; t0 < n_tasks; t0 += kPerPass) {
                const int task = t0 + sub;
                const bool active = task < n_tasks;
                const bool is_k = task == g, is_v = task == g + 1;
                const int head = task < g ? kvh * g + task : (is_k ? p.H + kvh : p.H + p.KV + kvh);
                float x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = 0.f;
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (active) {
                    raw = *reinterpret_cast<const uint4*>(p.qkv + (static_cast<int64_t>(cu0) * n_heads + head) * HD + c * 8);
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
                }
                if (active && is_v) {
                    *reinterpret_cast<uint4*>(newkv + HD + c * 8) = raw;
                    if (k_elem >= 0) *reinterpret_cast<uint4*>(p.cache + k_elem + static_cast<int64_t>(p.KV) * p.page_size * HD + c * 8) = raw;
                }
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
                for (int o = CPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (p.q_w != nullptr) {
                    const float inv = rsqrtf(ss / static_cast<float>(HD) + p.qk_eps);
                    const float* w = is_k ? p.k_w : p.q_w;
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = rnd<__nv_bfloat16>(rnd<__nv_bfloat16>(x[i] * inv) * w[c * 8 + i]);
                }
                float other[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, x[i], CPR / 2);
                if (!active || is_v) continue;
                uint4 packed;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    pw[i] = pack_bf16(x[2 * i] * cs[2 * i] + other[2 * i] * sn[2 * i], x[2 * i + 1] * cs[2 * i + 1] + other[2 * i + 1] * sn[2 * i + 1]);
                if (is_k) {
                    *reinterpret_cast<uint4*>(newkv + c * 8) = packed;
                    if (k_elem >= 0) *reinterpret_cast<uint4*>(p.cache + k_elem + c * 8) = packed;
                } else {
                    *reinterpret_cast<uint4*>(sm.q + swz<HD>(task, c)) = packed;
                }
            }
            for (int i = threadIdx.x; i < (16 - g) * CPR; i += kConsumers)    // rows without a query head are zero
                *reinterpret_cast<uint4*>(sm.q + swz<HD>(g + i / CPR, i % CPR)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(kThreads) : "memory");     // all queries; and the producer's barriers exist
            const int row_lo[2] = {key_lo, key_lo};
            const int row_hi[2] = {key_hi, key_hi};         // rows >= g hold zero queries and are never stored
            uint32_t qf[HD / 16][4];
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldmatrix_x4(qf[ks], sm.q + swz<HD>(lane & 15, ks * 2 + (lane >> 4)));
            for (int it = 0; it < n_tiles; ++it) {
                const int st = it % kDecStages;
                const int key0 = (tile_begin + it) * kBN + warp * 16;      // each warp takes 16 of the tile's 64 keys
                mbar_wait(full + st, (it / kDecStages) & 1, p.err);       // also when this warp's keys are all outside
                if (owns_pos && tile_begin + it == tile_of_pos && warp == (pos % kBN) / 16) {
                    // the token's own key and value are not in the cache's copy of this tile yet (they are being
                    // written by this very kernel): the warp that owns the row puts them into the tile
                    __nv_bfloat16* tile = sm.stages + st * Plan::kStageElems;
                    if (lane < 2 * CPR) {
                        const int which = lane / CPR, cc = lane % CPR;
                        *reinterpret_cast<uint4*>(tile + which * kBN * HD + kv_off(pos % kBN, cc)) =
                            *reinterpret_cast<const uint4*>(newkv + which * HD + cc * 8);
                    }
                    __syncwarp();
                }
                if (key0 <= key_hi && key0 + 15 >= key_lo) {
                    const __nv_bfloat16* sK = sm.stages + st * Plan::kStageElems;
                    __nv_bfloat16* sV = sm.stages + st * Plan::kStageElems + kBN * HD;
                    if (key0 + 15 > key_hi) clear_value_rows<HD>(sV, key_hi + 1 - (tile_begin + it) * kBN, warp * 16 + 15, lane);
                    float s[2][4];
                    qk_product<HD, 2>(s, qf, sK, warp * 16, lane);
                    if (key0 >= key_lo && key0 + 15 <= key_hi)
                        softmax_step<HD, 2, false>(s, o, m, l, key0, row_lo, row_hi, p.scale_log2, lane);
                    else
                        softmax_step<HD, 2, true>(s, o, m, l, key0, row_lo, row_hi, p.scale_log2, lane);
                    pv_product<HD, 2>(o, s, sV, warp * 16, lane);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + st);
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 1);
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 2);
    }
    if (fused && (n_tiles == 0 || warp == kConsumers / 32)) pdl_wait();    // every thread has waited before anything is written
    // The kernel behind this one may start now: its blocks arrive when most of this kernel's blocks have left their SMs, so
    // they spread evenly, and what they fetch ahead of their own wait overlaps the merge below.
    pdl_trigger();
    // combine the four warps through shared memory (the tiles are no longer needed); only the rows that hold a query
    __syncthreads();
    float* red_o = reinterpret_cast<float*>(sm.stages);                    // [4][16][HD]
    float* red_ml = red_o + 4 * 16 * HD;                                   // [4][16][2]
    // What the other blocks of the cluster send lies behind the new key and value, outside the tiles: a block that is
    // done may send while this one still computes.  recv_o [splits][share], recv_ml [splits][16][2], weight [16][16], sum [16].
    const int items = g * HD, share = (items + p.splits - 1) / p.splits;
    float* recv_o = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(sm.bars) + 64 + 2 * HD * sizeof(__nv_bfloat16));
    float* recv_ml = recv_o + p.splits * share;
    float* weight = recv_ml + p.splits * 32;
    float* row_sum = weight + 256;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = (lane >> 2) + half * 8;
        if (warp >= kConsumers / 32 || r >= g) continue;                   // the producer warp holds no results
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt)
            *reinterpret_cast<float2*>(red_o + (warp * 16 + r) * HD + dt * 8 + ((lane & 3) << 1)) = make_float2(o[dt][half * 2], o[dt][half * 2 + 1]);
        if ((lane & 3) == 0) *reinterpret_cast<float2*>(red_ml + (warp * 16 + r) * 2) = make_float2(m[half], l[half]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < items; i += kThreads) {
        const int r = i / HD, d = i % HD;
        float mw[4], mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) { mw[w] = red_ml[(w * 16 + r) * 2]; mm = fmaxf(mm, mw[w]); }
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = mw[w] == -INFINITY ? 0.f : exp2f(mw[w] - mm);
            acc += red_o[(w * 16 + r) * HD + d] * f;
            ll += red_ml[(w * 16 + r) * 2 + 1] * f;
        }
        if (p.splits == 1) {
            p.out[(static_cast<int64_t>(cu0) * p.H + kvh * g + r) * HD + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        } else if (p.cluster) {
            // The splits of this (request, kv head) are the blocks of one cluster.  Output element i is merged by block
            // i / share: this block's part of it goes straight into that block's shared memory, and its (maximum, sum)
            // of every row to all blocks.  Remote stores do not wait for anything; the cluster's barrier below makes
            // them visible.
            const int owner = i / share;
            st_cluster(recv_o + split * share + (i - owner * share), owner, acc);
            if (d < p.splits) {                                            // the row's first threads: one block each
                st_cluster(recv_ml + (split * 16 + r) * 2, d, mm);
                st_cluster(recv_ml + (split * 16 + r) * 2 + 1, d, ll);
            }
        } else {
            const int64_t base = ((static_cast<int64_t>(seq) * p.KV + kvh) * p.splits + split) * 16 + r;
            p.part_o[base * HD + d] = acc;
            if (d == 0) { p.part_ml[base * 2] = mm; p.part_ml[base * 2 + 1] = ll; }
        }
    }
    if (p.splits == 1 || !p.cluster) return;
    cluster_sync();
    // From here on every block reads its own shared memory only, so no second barrier is needed: nobody writes into a
    // block after the barrier, and nobody reads from it.
    // Row r's weights: sixteen neighbouring lanes hold the sixteen possible splits of the row, find the row's maximum
    // and the sum of the weighted sums by shuffles (a fixed tree: the same result in every block).
    // (whole warps walk the rows two at a time, so that every lane of a warp takes part in its shuffles)
    for (int r0 = warp * 2; r0 < g; r0 += (kThreads >> 5) * 2) {
        const int r = r0 + (lane >> 4), c = lane & 15;
        const bool has = r < g && c < p.splits;
        const float mc = has ? recv_ml[(c * 16 + r) * 2] : -INFINITY;
        const float lc = has ? recv_ml[(c * 16 + r) * 2 + 1] : 0.f;
        float mm = mc;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
        const float f = mc == -INFINITY ? 0.f : exp2f(mc - mm);
        float ll = lc * f;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
        if (r < g) {
            weight[r * 16 + c] = f;
            if (c == 0) row_sum[r] = ll;
        }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < share; j += kThreads) {
        const int i = split * share + j;
        if (i >= items) break;
        const int r = i / HD, d = i % HD;
        float acc = 0.f;
        for (int c = 0; c < p.splits; ++c) acc += recv_o[c * share + j] * weight[r * 16 + c];
        const float ll = row_sum[r];
        p.out[(static_cast<int64_t>(cu0) * p.H + kvh * g + r) * HD + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    }
}

template <int HD>
__global__ void attn_decode_merge_kernel(const AttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int cu0 = p.qkv != nullptr ? seq : p.cu_seqlens[seq];
    if (p.qkv == nullptr && p.cu_seqlens[seq + 1] - cu0 != 1) return;
    const int g = p.H / p.KV, kvh = h / g, r = h % g;
    const int64_t base = ((static_cast<int64_t>(seq) * p.KV + kvh) * p.splits) * 16 + r;
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, p.part_ml[(base + s * 16) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f, ll = 0.f;
        for (int s = 0; s < p.splits; ++s) {
            const float ms = p.part_ml[(base + s * 16) * 2];
            const float f = ms == -INFINITY ? 0.f : exp2f(ms - mm);
            acc += p.part_o[(base + s * 16) * HD + d] * f;
            ll += p.part_ml[(base + s * 16) * 2 + 1] * f;
        }
        p.out[(static_cast<int64_t>(cu0) * p.H + h) * HD + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    }
}

// ---- host side --------------------------------------------------------------------------------------------------

// A tensor map of one cache unit seen as [rows = pages * 2 * KV * page_size][head_dim] bf16, fetched in boxes of
// [box_rows][64 columns] with the 128-byte swizzle.
static int kv_tensor_map(CUtensorMap* out, const void* cache, int64_t rows, int hd, int box_rows) {
    return cached_bf16_map(out, cache, rows, hd, 64, box_rows);
}

template <int HD> constexpr size_t prefill_smem() { return SmemPlan<HD, kPreStages, 64>::kBytes; }
// Shared memory of the decode kernel for `g` query heads per kv head: the tiles (re-used for the four warps' results),
// the queries, the barriers, the new key and value, and what the cluster's blocks send one another (g * HD + 16 floats
// of output parts, then [16][16][2] maxima and sums, [16][16] weights, [16] row sums).
template <int HD> constexpr size_t decode_smem(int g = 16) {
    const size_t red = 1024 + static_cast<size_t>(4 * 16) * (HD + 2) * sizeof(float);
    const size_t plan = SmemPlan<HD, kDecStages, 16>::kBytes + 64 + 2 * HD * sizeof(__nv_bfloat16) +
                        (static_cast<size_t>(g) * HD + 16 + 512 + 256 + 16) * sizeof(float);
    return plan > red ? plan : red;
}

constexpr int kMaxClusterSplits = 16;       // 8 is the portable cluster size; up to 16 blocks with the opt-in attribute

// The decode kernel, then the merge kernel; or, with `cluster_merge` and 2 to 16 splits, the decode kernel alone with
// the splits of each (request, kv head) launched as one thread-block cluster that merges in shared memory.
template <int HD>
static int launch_decode(const CUtensorMap& map, AttnParams p, dim3 grid, dim3 mgrid, bool cluster_merge, cudaStream_t stream) {
    static bool set = false, wide_ok = false;
    if (!set) {
        cudaFuncSetAttribute(attn_decode_bf16_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<HD>());
        wide_ok = cudaFuncSetAttribute(attn_decode_bf16_kernel<HD>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        cudaGetLastError();
        set = true;
    }
    if (cluster_merge && p.splits > 1 && p.splits <= kMaxClusterSplits && (p.splits <= 8 || wide_ok)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = decode_smem<HD>(p.H / p.KV);
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = static_cast<unsigned>(p.splits);
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        // can the device hold a cluster of this size at all?  Asked once per size.
        static int fits[kMaxClusterSplits + 1] = {};              // 0: not asked yet, 1: yes, -1: no
        if (fits[p.splits] == 0) {
            int n = 0;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, attn_decode_bf16_kernel<HD>, &cfg);
            cudaGetLastError();
            fits[p.splits] = (e == cudaSuccess && n > 0) ? 1 : -1;
        }
        if (fits[p.splits] < 0) goto apart;
        p.cluster = 1;
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (pdl_enabled() && (p.qkv != nullptr ||
                              (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone))) {
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.numAttrs = 2;
        }
        cudaLaunchKernelEx(&cfg, attn_decode_bf16_kernel<HD>, map, p);
        return launch_status();
    }
apart:
    p.cluster = 0;
    if (p.splits > 1 && p.part_o == nullptr) return CVB_E_SCRATCH;
    launch_kernel(attn_decode_bf16_kernel<HD>, dim3(grid), dim3(kThreads), decode_smem<HD>(p.H / p.KV), stream, map, p);
    if (p.splits > 1) launch_kernel(attn_decode_merge_kernel<HD>, dim3(mgrid), dim3(HD), 0, stream, p);
    return launch_status();
}

static int check_common(int S, int H, int KV, int hd, int page_size, int table_width, int num_pages) {
    if (S <= 0 || H <= 0 || KV <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (H % KV) return CVB_E_SHAPE;
    if (hd != 64 && hd != 128) return CVB_E_UNSUPPORTED;
    if (H / KV > 16) return CVB_E_UNSUPPORTED;
    if (KV > 65535) return CVB_E_SIZE;
    // a TMA box is a whole page, or 64 rows of a larger page: pages of 16, 32, 64, 128, ... tokens
    if (page_size < 16 || (page_size & (page_size - 1)) != 0) return CVB_E_UNSUPPORTED;
    if (static_cast<int64_t>(num_pages) * 2 * KV * page_size > 2147483647LL) return CVB_E_SIZE;
    return CVB_OK;
}

}  // namespace cvb

using namespace cvb;

// Number of floats of scratch the decode kernel needs for a given launch.
extern "C" int64_t cvb_attn_decode_scratch_floats(int S, int KV, int hd, int splits) {
    if (splits <= 1) return 0;
    return static_cast<int64_t>(S) * KV * splits * 16 * (hd + 2);
}

static int fill_params(AttnParams& p, CUtensorMap& map, void* out, const void* q, const void* cache, const int* block_tables,
                       int table_width, const int* cu_seqlens, const int* positions, int S, int H, int KV, int hd,
                       int page_size, int window, float scale, int num_pages, int* err_flag) {
    const int rc = check_common(S, H, KV, hd, page_size, table_width, num_pages);
    if (rc != CVB_OK) return rc;
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2e; p.err = err_flag;
    p.box_rows = page_size < kBN ? page_size : kBN;
    return kv_tensor_map(&map, cache, static_cast<int64_t>(num_pages) * 2 * KV * page_size, hd, p.box_rows);
}

extern "C" int cvb_attn_prefill_bf16(void* out, const void* q, const void* cache, const int* block_tables,
                                     int table_width, const int* cu_seqlens, const int* positions, int S,
                                     int num_tiles, int H, int KV, int hd, int page_size, int window, float scale,
                                     int num_pages, int skip_single, int* err_flag, cudaStream_t stream) {
    if (num_tiles == 0) return CVB_OK;
    if (num_tiles < 0) return CVB_E_SIZE;
    AttnParams p{};
    CUtensorMap map;
    const int rc = fill_params(p, map, out, q, cache, block_tables, table_width, cu_seqlens, positions, S, H, KV, hd,
                               page_size, window, scale, num_pages, err_flag);
    if (rc != CVB_OK) return rc;
    dim3 grid(static_cast<unsigned>(num_tiles), static_cast<unsigned>(KV));
    if (hd == 128) {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_bf16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem<128>()); set = true; }
        launch_kernel(attn_prefill_bf16_kernel<128>, dim3(grid), dim3(kThreads), prefill_smem<128>(), stream, map, p, skip_single);
    } else {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_bf16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem<64>()); set = true; }
        launch_kernel(attn_prefill_bf16_kernel<64>, dim3(grid), dim3(kThreads), prefill_smem<64>(), stream, map, p, skip_single);
    }
    return launch_status();
}

extern "C" int cvb_attn_decode_bf16(void* out, const void* q, const void* cache, const int* block_tables,
                                    int table_width, const int* cu_seqlens, const int* positions, int S, int H,
                                    int KV, int hd, int page_size, int window, float scale, int num_pages,
                                    int splits, float* scratch, int64_t scratch_floats, int cluster_merge, int* err_flag,
                                    cudaStream_t stream) {
    if (splits < 1 || splits > 65535) return CVB_E_SIZE;
    AttnParams p{};
    CUtensorMap map;
    const int rc = fill_params(p, map, out, q, cache, block_tables, table_width, cu_seqlens, positions, S, H, KV, hd,
                               page_size, window, scale, num_pages, err_flag);
    if (rc != CVB_OK) return rc;
    if (cluster_merge && splits > kMaxClusterSplits) cluster_merge = 0;
    if (splits > 1 && !cluster_merge && (scratch == nullptr || scratch_floats < cvb_attn_decode_scratch_floats(S, KV, hd, splits)))
        return CVB_E_SCRATCH;
    p.splits = splits;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + static_cast<int64_t>(S) * KV * splits * 16 * hd : nullptr;
    dim3 grid(static_cast<unsigned>(S), static_cast<unsigned>(KV), static_cast<unsigned>(splits));
    dim3 mgrid(static_cast<unsigned>(S), static_cast<unsigned>(H));
    if (hd == 128) return launch_decode<128>(map, p, grid, mgrid, cluster_merge != 0, stream);
    return launch_decode<64>(map, p, grid, mgrid, cluster_merge != 0, stream);
}

// Decode attention straight from the projection's output: per-head norm and rotation of the queries, norm, rotation and
// cache write of the new key, cache write of the new value, and the attention itself in one kernel.  Every request brings
// exactly one token (T = S, token s belongs to request s; `cu_seqlens` is not read).  `qkv` is [T, H + 2 KV, hd]; `slots[t]` is the cache slot of token t; `q_w`/`k_w` are the per-head norm weights (both null: no
// norm) and `cos_t`/`sin_t` the rotation tables over the whole head in rotate-half pairing (both null: no rotation).
extern "C" int cvb_attn_decode_fused_bf16(void* out, const void* qkv, void* cache, const int* block_tables, int table_width,
                                          const int* cu_seqlens, const int* positions, const int* slots, int S, int H,
                                          int KV, int hd, int page_size, int window, float scale, int num_pages,
                                          int splits, float* scratch, int64_t scratch_floats, const float* q_w,
                                          const float* k_w, float qk_eps, const float* cos_t, const float* sin_t,
                                          int max_pos, int* err_flag, cudaStream_t stream) {
    if (splits < 1 || splits > 65535) return CVB_E_SIZE;
    if (qkv == nullptr || slots == nullptr || (q_w == nullptr) != (k_w == nullptr)) return CVB_E_SHAPE;
    if ((cos_t == nullptr) != (sin_t == nullptr) || (cos_t != nullptr && max_pos <= 0)) return CVB_E_SHAPE;
    auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(qkv) || !al(cos_t) || !al(sin_t) || !al(cache)) return CVB_E_ALIGN;
    AttnParams p{};
    CUtensorMap map;
    const int rc = fill_params(p, map, out, qkv, cache, block_tables, table_width, cu_seqlens, positions, S, H, KV, hd,
                               page_size, window, scale, num_pages, err_flag);
    if (rc != CVB_OK) return rc;
    const bool cluster = splits <= kMaxClusterSplits;
    if (splits > 1 && !cluster && (scratch == nullptr || scratch_floats < cvb_attn_decode_scratch_floats(S, KV, hd, splits)))
        return CVB_E_SCRATCH;
    p.splits = splits;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + static_cast<int64_t>(S) * KV * splits * 16 * hd : nullptr;
    p.qkv = (const __nv_bfloat16*)qkv; p.q_w = q_w; p.k_w = k_w; p.qk_eps = qk_eps; p.cos_t = cos_t; p.sin_t = sin_t;
    p.max_pos = max_pos; p.slots = slots; p.cache = (__nv_bfloat16*)cache;
    p.cache_elems = static_cast<int64_t>(num_pages) * 2 * KV * page_size * hd;
    dim3 grid(static_cast<unsigned>(S), static_cast<unsigned>(KV), static_cast<unsigned>(splits));
    dim3 mgrid(static_cast<unsigned>(S), static_cast<unsigned>(H));
    if (hd == 128) return launch_decode<128>(map, p, grid, mgrid, cluster, stream);
    return launch_decode<64>(map, p, grid, mgrid, cluster, stream);
}

// ---- split-KV decode attention without any allocation ---------------------------------------------------------------
//
// cvb_attn_decode_bf16_static is cvb_attn_decode_bf16 for callers that must not allocate device memory while they
// run: code inside a real-time or safety-reviewed loop that may not call cudaMalloc, a plug-in that lives under
// another program's memory budget, a host that has handed the whole device to a pool it cannot ask.  The caller
// still passes queries, pages, tables and the output; only the scratch for the partial results of the splits, which
// the other entry point takes as an argument, lives here in a file-scope device array of kStaticScratchFloats
// floats (8 MiB).  Every GPU that loads this library holds that array until the process exits.
//
// The array's name is a host-side stand-in in host code, not a device address; the kernels need the address.  It is
// looked up with cudaGetSymbolAddress once per device, with that device current, at the first call on that device.
// That first call also sets kernel attributes, so make it before any stream capture starts.
//
// A launch whose partial results do not fit (requests * kv heads * splits * 16 * (head_dim + 2) floats) is refused
// with CVB_E_SCRATCH; nothing is launched.  No cudaMalloc, cudaFree or allocating library routine is called, and
// the tensor map is built on the stack at every call.  All calls share the one array and it keeps the last
// call's contents.  Nothing in it has to start at zero: every block writes the partial results that the merge kernel
// of the same call reads.  Calls that overlap on the GPU (two streams, or two host threads on different streams)
// race on it; keep calls that use this entry point on one stream, or order them with events.
namespace cvb {

constexpr int64_t kStaticScratchFloats = int64_t{1} << 21;
static __device__ __align__(256) float g_static_decode_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_ptr[kMaxDevices] = {};
static std::mutex g_static_scratch_mu;

// Device address of the scratch array on the current device; looked up once per device.
static int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return CVB_E_SIZE;
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (g_static_scratch_ptr[dev] == nullptr) {
        float* ptr = nullptr;
        // a failed call leaves its error behind in the runtime; it is taken out here (cudaGetLastError), so that the next
        // launcher's status check does not report it against an unrelated kernel
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_decode_scratch);
        if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
        if (ptr == nullptr) return CVB_E_SCRATCH;
        e = cudaFuncSetAttribute(attn_decode_bf16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<128>());
        if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
        e = cudaFuncSetAttribute(attn_decode_bf16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<64>());
        if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return CVB_OK;
}

}  // namespace cvb

extern "C" int64_t cvb_attn_decode_static_scratch_floats() { return cvb::kStaticScratchFloats; }

extern "C" int cvb_attn_decode_bf16_static(void* out, const void* q, const void* cache, const int* block_tables,
                                           int table_width, const int* cu_seqlens, const int* positions, int S, int H,
                                           int KV, int hd, int page_size, int window, float scale, int num_pages,
                                           int splits, int* err_flag, cudaStream_t stream) {
    if (splits < 1 || splits > 65535) return CVB_E_SIZE;
    int rc = check_common(S, H, KV, hd, page_size, table_width, num_pages);
    if (rc != CVB_OK) return rc;
    if (cvb_attn_decode_scratch_floats(S, KV, hd, splits) > kStaticScratchFloats) return CVB_E_SCRATCH;
    float* scratch = nullptr;
    rc = static_scratch_for_current_device(&scratch);
    if (rc != CVB_OK) return rc;

    AttnParams p{};
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2e; p.err = err_flag;
    p.box_rows = page_size < kBN ? page_size : kBN;
    p.splits = splits;
    p.part_o = scratch;
    p.part_ml = scratch + static_cast<int64_t>(S) * KV * splits * 16 * hd;

    // the tensor map is encoded into a local variable: no table, no heap
    CUtensorMap map;
    rc = encode_bf16_map(&map, cache, static_cast<int64_t>(num_pages) * 2 * KV * page_size, hd, 64, p.box_rows);
    if (rc != CVB_OK) return rc;

    dim3 grid(static_cast<unsigned>(S), static_cast<unsigned>(KV), static_cast<unsigned>(splits));
    dim3 mgrid(static_cast<unsigned>(S), static_cast<unsigned>(H));
    if (hd == 128) {
        launch_kernel(attn_decode_bf16_kernel<128>, dim3(grid), dim3(kThreads), decode_smem<128>(H / KV), stream, map, p);
        if (splits > 1) launch_kernel(attn_decode_merge_kernel<128>, dim3(mgrid), dim3(128), 0, stream, p);
    } else {
        launch_kernel(attn_decode_bf16_kernel<64>, dim3(grid), dim3(kThreads), decode_smem<64>(H / KV), stream, map, p);
        if (splits > 1) launch_kernel(attn_decode_merge_kernel<64>, dim3(mgrid), dim3(64), 0, stream, p);
    }
    return launch_status();
}
