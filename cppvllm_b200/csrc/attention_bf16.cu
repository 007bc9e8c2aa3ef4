// Tensor-core attention over the paged cache for bf16, head sizes 64 and 128.
//
//   cvb_attn_prefill_bf16  prompt portions (requests with more than one token in the step): flash attention with a
//                          causal offset, reading ALL keys (earlier portions' and the step's own) from the pages.
//   cvb_attn_decode_bf16   single decoded tokens: the key range of every (request, kv head) is cut into `splits`
//                          chunks that run in parallel; partial (max, sum, output) triples go to scratch memory
//                          and cvb_attn_decode_merge (launched by the same entry point) combines them.
//
// Both kernels put the query heads that share a kv head next to each other in the M dimension of the matrix
// product (row r = token r / g, head kvh * g + r % g), so a key/value tile is loaded once for the whole group.
// Scores, softmax statistics and the output accumulator are float; probabilities are rounded to bf16 for the
// second product, as flash attention does.  Formulas as in attention_general.cu (reference
// kernels/paged_attention.cu:89-359: scale * q.k, keys lo..p, online softmax, o = sum p v / l).
//
// Tiles move with cp.async (16-byte chunks; rows beyond the request's length are zero-filled and never read from
// memory); shared-memory rows are XOR-swizzled in 16-byte chunks so that ldmatrix is conflict-free.  The matrix
// products are mma.sync.m16n8k16 (bf16 in, float accumulate).
#include "common.cuh"

namespace cvb {

constexpr int kBN = 64;                 // keys per tile
constexpr int kThreads = 128;           // 4 warps
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int n = valid ? 16 : 0;       // src-size 0: nothing is read, the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

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

// element offset of 16-byte chunk `c` of row `r` in a swizzled tile whose rows hold HD bf16
template <int HD> __device__ __forceinline__ int swz(int r, int c) { return r * HD + ((c ^ (r & 7)) << 3); }

struct AttnParams {
    __nv_bfloat16* out;                 // [T, H, HD]
    const __nv_bfloat16* q;             // [T, H, HD]
    const __nv_bfloat16* cache;         // [pages, 2, KV, page_size, HD]
    const int* block_tables;            // [S, table_width]
    const int* cu_seqlens;              // [S + 1]
    const int* positions;               // [T]
    int table_width, S, H, KV, page_size, window, num_pages;
    float scale_log2;                   // scale * log2(e)
    int* err;
    // decode only
    float* part_o;                      // [S, KV, splits, 16, HD]
    float* part_ml;                     // [S, KV, splits, 16, 2]
    int splits;
};

// Loads keys [key0, key0 + 64) of one kv head into a swizzled tile: `which` = 0 for K, 1 for V.
template <int HD>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* tile, const AttnParams& p, const int* table, int kvh,
                                             int which, int key0, int key_lo, int key_hi) {
    constexpr int CPR = HD / 8;                         // chunks per row
    for (int i = threadIdx.x; i < kBN * CPR; i += kThreads) {
        const int r = i / CPR, c = i % CPR;
        const int j = key0 + r;
        bool valid = j >= key_lo && j <= key_hi;
        const __nv_bfloat16* src = p.cache;
        if (valid) {
            const int slot = j / p.page_size;
            const int page = slot < p.table_width ? table[slot] : -1;
            if (page < 0 || page >= p.num_pages) {
                atomicExch(p.err, 4);
                valid = false;
            } else {
                src = p.cache + ((((static_cast<int64_t>(page) * 2 + which) * p.KV + kvh) * p.page_size + j % p.page_size) * HD + c * 8);
            }
        }
        cp_async16(tile + swz<HD>(r, c), src, valid);
    }
}

// One warp: S[16 x NK*8] = Q[16 x HD] * K^T over NK/2 groups of 16 keys starting at tile row `krow0`.
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
            ldmatrix_x4(b, sK + swz<HD>(r, c));
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
            ldmatrix_x4_trans(b, sV + swz<HD>(r, c));
            mma_bf16(o[dp * 2], a, b[0], b[1]);
            mma_bf16(o[dp * 2 + 1], a, b[2], b[3]);
        }
    }
}

// Masks the score tile, updates the running max and sum of the warp's two rows per thread, rescales the output
// accumulator and turns scores into probabilities.  Column n of the tile is key `key0 + n`.
template <int HD, int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[HD / 8][4], float (&m)[2], float (&l)[2],
                                             int key0, const int (&row_lo)[2], const int (&row_hi)[2],
                                             float scale_log2, int lane) {
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int half = e >> 1;
            const int j = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
            const bool ok = j >= row_lo[half] && j <= row_hi[half];
            s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
            tile_max[half] = fmaxf(tile_max[half], s[nt][e]);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        tile_max[half] = fmaxf(tile_max[half], __shfl_xor_sync(0xffffffffu, tile_max[half], 1));
        tile_max[half] = fmaxf(tile_max[half], __shfl_xor_sync(0xffffffffu, tile_max[half], 2));
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const float m_new = fmaxf(m[half], tile_max[half]);
        m_use[half] = m_new == -INFINITY ? 0.f : m_new;
        corr[half] = m[half] == -INFINITY ? 0.f : exp2f(m[half] - m_use[half]);
        m[half] = m_new;
    }
    float tile_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int half = e >> 1;
            const float pr = exp2f(s[nt][e] - m_use[half]);       // exp2(-inf) = 0 for excluded keys
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

// ---- prefill ---------------------------------------------------------------------------------------------------

template <int HD>
__global__ void __launch_bounds__(kThreads)
attn_prefill_bf16_kernel(const AttnParams p, const int skip_single) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [64][HD]
    __nv_bfloat16* sK = sQ + 64 * HD;                                      // [2][64][HD]
    __nv_bfloat16* sV = sK + 2 * kBN * HD;                                 // [2][64][HD]
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
    const int tile_begin = key_lo / kBN, tile_end = key_hi / kBN;

    // Q tile: row r = (token r / g, head kvh * g + r % g)
    for (int i = threadIdx.x; i < 64 * CPR; i += kThreads) {
        const int r = i / CPR, c = i % CPR;
        const int tok = r / g;
        const bool valid = tok < n_tok;
        const __nv_bfloat16* src = valid ? p.q + ((static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * HD + c * 8) : p.q;
        cp_async16(sQ + swz<HD>(r, c), src, valid);
    }
    load_kv_tile<HD>(sK, p, table, kvh, 0, tile_begin * kBN, key_lo, key_hi);
    load_kv_tile<HD>(sV, p, table, kvh, 1, tile_begin * kBN, key_lo, key_hi);
    cp_async_commit();

    // the two rows this thread owns in the warp's 16-row slab
    int row_lo[2], row_hi[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int tok = r / g;
        if (tok < n_tok) {
            const int pos = p.positions[cu0 + q0 + tok];
            row_hi[half] = pos;
            row_lo[half] = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        } else {
            row_hi[half] = -1;                          // no key passes lo <= j <= hi
            row_lo[half] = 0;
        }
    }

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int kt = tile_begin; kt <= tile_end; ++kt) {
        const int buf = (kt - tile_begin) & 1;
        if (kt + 1 <= tile_end) {
            load_kv_tile<HD>(sK + (buf ^ 1) * kBN * HD, p, table, kvh, 0, (kt + 1) * kBN, key_lo, key_hi);
            load_kv_tile<HD>(sV + (buf ^ 1) * kBN * HD, p, table, kvh, 1, (kt + 1) * kBN, key_lo, key_hi);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (kt == tile_begin) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldmatrix_x4(qf[ks], sQ + swz<HD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
        }
        // a warp whose rows all end before this tile has nothing to add (causal)
        const int warp_hi = p.positions[cu0 + q0 + min(n_tok - 1, (warp * 16 + 15) / g)];
        if (kt * kBN <= warp_hi && warp * 16 < n_tok * g) {
            float s[8][4];
            qk_product<HD, 8>(s, qf, sK + buf * kBN * HD, 0, lane);
            softmax_step<HD, 8>(s, o, m, l, kt * kBN, row_lo, row_hi, p.scale_log2, lane);
            pv_product<HD, 8>(o, s, sV + buf * kBN * HD, 0, lane);
        }
        __syncthreads();
    }
    cp_async_wait<0>();

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
attn_decode_bf16_kernel(const AttnParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [16][HD]
    __nv_bfloat16* sK = sQ + 16 * HD;                                      // [stages][64][HD]
    __nv_bfloat16* sV = sK + kDecStages * kBN * HD;                        // [stages][64][HD]
    constexpr int CPR = HD / 8;
    const int g = p.H / p.KV;
    const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cu0 = p.cu_seqlens[seq];
    if (p.cu_seqlens[seq + 1] - cu0 != 1) return;                          // not a single decoded token
    const int pos = p.positions[cu0];
    const int key_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int key_hi = pos;
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int first_tile = key_lo / kBN, n_tiles = key_hi / kBN - first_tile + 1;
    const int per_split = (n_tiles + p.splits - 1) / p.splits;
    const int tile_begin = first_tile + split * per_split;
    const int tile_end = min(first_tile + n_tiles, tile_begin + per_split) - 1;      // inclusive; may be < begin

    float o[HD / 8][4];
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) { o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (tile_begin <= tile_end) {
        for (int i = threadIdx.x; i < 16 * CPR; i += kThreads) {
            const int r = i / CPR, c = i % CPR;
            const bool valid = r < g;
            const __nv_bfloat16* src = valid ? p.q + ((static_cast<int64_t>(cu0) * p.H + kvh * g + r) * HD + c * 8) : p.q;
            cp_async16(sQ + swz<HD>(r, c), src, valid);
        }
#pragma unroll
        for (int st = 0; st < kDecStages - 1; ++st) {
            if (tile_begin + st <= tile_end) {
                load_kv_tile<HD>(sK + st * kBN * HD, p, table, kvh, 0, (tile_begin + st) * kBN, key_lo, key_hi);
                load_kv_tile<HD>(sV + st * kBN * HD, p, table, kvh, 1, (tile_begin + st) * kBN, key_lo, key_hi);
            }
            cp_async_commit();
        }
        const int row_lo[2] = {key_lo, key_lo};
        const int row_hi2[2] = {(lane >> 2) < g ? key_hi : -1, ((lane >> 2) + 8) < g ? key_hi : -1};   // rows >= g carry no head
        uint32_t qf[HD / 16][4];
        for (int kt = tile_begin; kt <= tile_end; ++kt) {
            const int it = kt - tile_begin;
            const int buf = it % kDecStages;
            const int nxt = kt + kDecStages - 1;
            if (nxt <= tile_end) {
                const int nb = (it + kDecStages - 1) % kDecStages;
                load_kv_tile<HD>(sK + nb * kBN * HD, p, table, kvh, 0, nxt * kBN, key_lo, key_hi);
                load_kv_tile<HD>(sV + nb * kBN * HD, p, table, kvh, 1, nxt * kBN, key_lo, key_hi);
            }
            cp_async_commit();
            cp_async_wait<kDecStages - 1>();
            __syncthreads();
            if (it == 0) {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    ldmatrix_x4(qf[ks], sQ + swz<HD>(lane & 15, ks * 2 + (lane >> 4)));
            }
            // each warp takes 16 of the tile's 64 keys
            float s[2][4];
            qk_product<HD, 2>(s, qf, sK + buf * kBN * HD, warp * 16, lane);
            softmax_step<HD, 2>(s, o, m, l, kt * kBN + warp * 16, row_lo, row_hi2, p.scale_log2, lane);
            pv_product<HD, 2>(o, s, sV + buf * kBN * HD, warp * 16, lane);
            __syncthreads();
        }
        cp_async_wait<0>();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 1);
        l[half] += __shfl_xor_sync(0xffffffffu, l[half], 2);
    }
    // combine the four warps through shared memory (the tiles are no longer needed)
    __syncthreads();
    float* red_o = reinterpret_cast<float*>(smem_raw);                     // [4][16][HD]
    float* red_ml = red_o + 4 * 16 * HD;                                   // [4][16][2]
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = (lane >> 2) + half * 8;
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
            const int d = dt * 8 + ((lane & 3) << 1);
            red_o[(warp * 16 + r) * HD + d] = o[dt][half * 2];
            red_o[(warp * 16 + r) * HD + d + 1] = o[dt][half * 2 + 1];
        }
        if ((lane & 3) == 0) {
            red_ml[(warp * 16 + r) * 2] = m[half];
            red_ml[(warp * 16 + r) * 2 + 1] = l[half];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < g * HD; i += kThreads) {
        const int r = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_ml[(w * 16 + r) * 2]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            acc += red_o[(w * 16 + r) * HD + d] * f;
            ll += red_ml[(w * 16 + r) * 2 + 1] * f;
        }
        if (p.splits == 1) {
            p.out[(static_cast<int64_t>(cu0) * p.H + kvh * g + r) * HD + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        } else {
            const int64_t base = ((static_cast<int64_t>(seq) * p.KV + kvh) * p.splits + split) * 16 + r;
            p.part_o[base * HD + d] = acc;
            if (d == 0) { p.part_ml[base * 2] = mm; p.part_ml[base * 2 + 1] = ll; }
        }
    }
}

template <int HD>
__global__ void attn_decode_merge_kernel(const AttnParams p) {
    const int seq = blockIdx.x, h = blockIdx.y;
    const int cu0 = p.cu_seqlens[seq];
    if (p.cu_seqlens[seq + 1] - cu0 != 1) return;
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

template <int HD> constexpr size_t prefill_smem() { return static_cast<size_t>(64 + 4 * kBN) * HD * sizeof(__nv_bfloat16); }
template <int HD> constexpr size_t decode_smem() {
    const size_t tiles = static_cast<size_t>(16 + 2 * kDecStages * kBN) * HD * sizeof(__nv_bfloat16);
    const size_t red = static_cast<size_t>(4 * 16) * (HD + 2) * sizeof(float);
    return tiles > red ? tiles : red;
}

static int check_common(int S, int H, int KV, int hd, int page_size, int table_width, int num_pages) {
    if (S <= 0 || H <= 0 || KV <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (H % KV) return CVB_E_SHAPE;
    if (hd != 64 && hd != 128) return CVB_E_UNSUPPORTED;
    if (H / KV > 16) return CVB_E_UNSUPPORTED;
    if (KV > 65535) return CVB_E_SIZE;
    return CVB_OK;
}

}  // namespace cvb

using namespace cvb;

// Number of floats of scratch the decode kernel needs for a given launch.
extern "C" int64_t cvb_attn_decode_scratch_floats(int S, int KV, int hd, int splits) {
    if (splits <= 1) return 0;
    return static_cast<int64_t>(S) * KV * splits * 16 * (hd + 2);
}

extern "C" int cvb_attn_prefill_bf16(void* out, const void* q, const void* cache, const int* block_tables,
                                     int table_width, const int* cu_seqlens, const int* positions, int S,
                                     int num_tiles, int H, int KV, int hd, int page_size, int window, float scale,
                                     int num_pages, int skip_single, int* err_flag, cudaStream_t stream) {
    if (num_tiles == 0) return CVB_OK;
    const int rc = check_common(S, H, KV, hd, page_size, table_width, num_pages);
    if (rc != CVB_OK) return rc;
    if (num_tiles < 0) return CVB_E_SIZE;
    AttnParams p{};
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2e; p.err = err_flag;
    dim3 grid(static_cast<unsigned>(num_tiles), static_cast<unsigned>(KV));
    if (hd == 128) {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_bf16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem<128>()); set = true; }
        attn_prefill_bf16_kernel<128><<<grid, kThreads, prefill_smem<128>(), stream>>>(p, skip_single);
    } else {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_bf16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem<64>()); set = true; }
        attn_prefill_bf16_kernel<64><<<grid, kThreads, prefill_smem<64>(), stream>>>(p, skip_single);
    }
    return launch_status();
}

extern "C" int cvb_attn_decode_bf16(void* out, const void* q, const void* cache, const int* block_tables,
                                    int table_width, const int* cu_seqlens, const int* positions, int S, int H,
                                    int KV, int hd, int page_size, int window, float scale, int num_pages,
                                    int splits, float* scratch, int64_t scratch_floats, int* err_flag,
                                    cudaStream_t stream) {
    const int rc = check_common(S, H, KV, hd, page_size, table_width, num_pages);
    if (rc != CVB_OK) return rc;
    if (splits < 1 || splits > 65535) return CVB_E_SIZE;
    if (splits > 1 && (scratch == nullptr || scratch_floats < cvb_attn_decode_scratch_floats(S, KV, hd, splits)))
        return CVB_E_SCRATCH;
    AttnParams p{};
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2e; p.err = err_flag; p.splits = splits;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + static_cast<int64_t>(S) * KV * splits * 16 * hd : nullptr;
    dim3 grid(static_cast<unsigned>(S), static_cast<unsigned>(KV), static_cast<unsigned>(splits));
    dim3 mgrid(static_cast<unsigned>(S), static_cast<unsigned>(H));
    if (hd == 128) {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_decode_bf16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<128>()); set = true; }
        attn_decode_bf16_kernel<128><<<grid, kThreads, decode_smem<128>(), stream>>>(p);
        if (splits > 1) attn_decode_merge_kernel<128><<<mgrid, 128, 0, stream>>>(p);
    } else {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_decode_bf16_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<64>()); set = true; }
        attn_decode_bf16_kernel<64><<<grid, kThreads, decode_smem<64>(), stream>>>(p);
        if (splits > 1) attn_decode_merge_kernel<64><<<mgrid, 64, 0, stream>>>(p);
    }
    return launch_status();
}
