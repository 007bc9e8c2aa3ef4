// Flash attention for prompt portions on the fifth-generation tensor cores (tcgen05), bf16, head sizes 64 and 128,
// over the paged cache with a causal offset (and an optional window).  Same arithmetic as attention_bf16.cu (reference
// kernels/paged_attention.cu:89-359: scale * q.k over keys lo..p, online softmax in float, o = sum p v / l).
//
// One block owns 256 query rows of one kv head as two tiles X = A, B of 128 rows: the query heads that share the kv head
// are packed next to each other (row r of a tile = token r / g, head kvh * g + r % g), so a key/value tile is fetched
// once for the whole group and for both query tiles.  Keys are walked in tiles of 128.  The tensor core alternates
// between the two query tiles: while the softmax of one runs, the products of the other do.  Roles, by warp:
//   warp 0     producer: one lane per TMA box (a page or 64 keys, times 64-column half, times K and V; 128-byte swizzle),
//              two stages, each with the keys of tile j + 1 and the values of tile j (what one round of the tensor core
//              reads), so a round costs the issuing thread one wait and one commit for its operands; the block-table
//              reads of a load are in flight together;
//   warp 1     allocates 512 columns of tensor memory; one thread issues, per key tile j and query tile X,
//                  PV_j(X)    = P_j(X) V_j        (M 128, N = head size, K 128; P from tensor memory, V MN-major)
//                  S_{j+1}(X) = Q(X) K_{j+1}^T    (M 128, N 128, K = head size; both operands K-major)
//              PV_j(X) accumulates into O(X) in tensor memory; P_j(X) lies over the first half of S_j(X), where the
//              softmax threads put it, so S_{j+1}(X) follows PV_j(X) in the tensor core's queue;
//   warps 2-3  idle (they fill the first warpgroup, which hands its registers to the other two with setmaxnreg);
//   warps 4-7  softmax of tile A, warps 8-11 of tile B: one thread per query row.  A thread reads its row of S (128
//              floats) with tcgen05.ld, exponentiates against a reference maximum and writes the row of P as bf16 back
//              into tensor memory with tcgen05.st.  The output accumulator stays in tensor memory; it is rescaled (read,
//              multiplied, written back by the row's thread) only when the running maximum of some row of the warp has
//              grown by more than 2^8 since the reference was set, which happens in the first tiles and then hardly
//              ever.  The result is exact: the same reference scales P and the row sum.
// A grid of few query blocks with many key tiles each (a portion behind a long context) leaves SMs idle, so the launcher
// may allow a query block's key tiles to be shared out among up to eight blocks ("pieces"); each leaves its unnormalised
// rows, reference maxima and sums in global memory, and attn_prefill_merge_kernel adds them up in the order of the pieces.
// Tensor memory columns: S(A) 0..127, S(B) 128..255, O(A) 256.., O(B) 256 + head size...
// Buffers are handed over with mbarriers: TMA transaction counts, tcgen05.commit arrivals from the tensor core, and
// plain arrivals from the softmax threads.  Every wait is bounded by a cycle count; a wait that runs out records
// error 5 and the block runs on to its end (tensor memory is always given back).
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace cvb {

constexpr int kTM = 128;                      // query rows per block
constexpr int kTN = 128;                      // keys per tile
constexpr int kStages = 2;                    // each holds the keys of tile j + 1 and the values of tile j
constexpr float kLog2eF = 1.4426950408889634f;

// element offset of 16-byte chunk c of row r in a [128 rows][HD] tile stored as HD/64 halves of [128][64], swizzled
__device__ __forceinline__ int tile_off(int r, int c) { return ((c >> 3) << 13) + (r << 6) + (((c & 7) ^ (r & 7)) << 3); }

struct TcAttnParams {
    __nv_bfloat16* out;
    const __nv_bfloat16* q;
    const int* block_tables;
    const int* cu_seqlens;
    const int* positions;
    int table_width, S, H, KV, page_size, window, num_pages, box_rows;
    float scale_log2;
    int* err;
    // A query block's key tiles may be shared out among up to `pieces` blocks (see the kernel's comment).
    int pieces, min_rounds;
    float* part_o;            // [query block * kv head * pieces][2 query tiles][HD][128 rows]
    float* part_ml;           // [query block * kv head * pieces][2 query tiles][maximum | sum][128 rows]
    int* piece_counts;        // [query block * kv head]: into how many pieces the block was cut (written by piece 0)
};

constexpr int kTcThreads = 128 + 256;         // one warpgroup of helpers (two warps idle), one warpgroup per query tile

template <int HD>
struct TcSmem {
    static constexpr int kTile = 128 * HD * 2;
    static constexpr int kNumBars = 2 * kStages + 2 + 2 + 2;
    static constexpr size_t kBytes = static_cast<size_t>(kTile) * (2 + 2 * kStages) + kNumBars * 8 + 16;
};

constexpr float kRescaleStep = 8.f;            // log2 of the growth of a row's maximum that forces a rescale

template <int HD>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap kv_map, const TcAttnParams p, const int skip_single) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using L = TcSmem<HD>;
    pdl_trigger();
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(p.err, 6);
        return;
    }
    unsigned char* sQ = smem_raw;                                   // two tiles
    unsigned char* sKV = sQ + 2 * L::kTile;                         // stage s: keys at (2 s) tiles, values at (2 s + 1) tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + 2 * kStages * L::kTile);
    uint64_t* kv_full = bars;                      // [2]  TMA: the stage's keys and values have landed
    uint64_t* kv_empty = kv_full + kStages;        // [2]  tensor core: the products that read the stage are done
    uint64_t* s_ready = kv_empty + kStages;        // [2 tiles]  tensor core: S_j(X) and everything issued before it is done
    uint64_t* p_ready = s_ready + 2;               // [2 tiles]  128 softmax threads: P_j(X) is in tensor memory
    uint64_t* o_done = p_ready + 2;                // [2 tiles]  tensor core: the last PV(X) is done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = p.H / p.KV;
    const int tok_per_tile = kTM / g;
    const int tok_per_block = 2 * tok_per_tile;
    const int kvh = blockIdx.x;
    constexpr int CPR = HD / 8;

    int seq = -1, q0 = 0, q_len = 0, cu0 = 0;
    // Blocks are handed out with the kv head running fastest, then the query block, long ones (late in their request)
    // first, then the piece: all first pieces start before any second piece, and the blocks that find nothing to do
    // (a piece beyond the number its query block is cut into) come last within their piece.
    const int block_id = gridDim.y - 1 - blockIdx.y, piece = blockIdx.z;
    {
        // Which request the query block belongs to: the lanes of a warp take a request each (every warp does the same),
        // count its query blocks, add them up with shuffles and see whose range holds block_id: one trip to memory
        // for up to 32 requests instead of one per request.
        int before = 0;
        for (int s0 = 0; s0 < p.S && seq < 0; s0 += 32) {
            const int s = s0 + lane;
            int a = 0, n = 0;
            if (s < p.S) { a = p.cu_seqlens[s]; n = p.cu_seqlens[s + 1] - a; }
            const int tiles = (s < p.S && !(skip_single && n == 1)) ? (n + tok_per_block - 1) / tok_per_block : 0;
            int upto = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, upto, o);
                if (lane >= o) upto += v;
            }
            const int first = before + upto - tiles;
            const unsigned hit = __ballot_sync(0xffffffffu, tiles > 0 && block_id >= first && block_id < first + tiles);
            if (hit) {
                const int src = __ffs(hit) - 1;
                seq = s0 + src;
                q0 = (block_id - __shfl_sync(0xffffffffu, first, src)) * tok_per_block;
                q_len = __shfl_sync(0xffffffffu, n, src);
                cu0 = __shfl_sync(0xffffffffu, a, src);
            }
            before += __shfl_sync(0xffffffffu, upto, 31);
        }
    }
    if (seq < 0) return;
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    int n_tok[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) n_tok[x] = max(0, min(tok_per_tile, q_len - q0 - x * tok_per_tile));
    // r / g for r < 256 without a division (g <= 16): exact with this multiplier
    const uint32_t g_mul = ((1u << 20) + g - 1) / g;
    auto row_tok = [&](int r) { return static_cast<int>((static_cast<uint32_t>(r) * g_mul) >> 20); };
    // The positions of each query tile's first and last token are asked for here and used further down: they are a step
    // input, in place before the first kernel of the step started, so they may be read ahead of griddepcontrol.wait.
    int first_pos[2] = {0, 0}, last_pos[2] = {0, 0};
    const int seq_last = p.positions[cu0 + q_len - 1];              // the request's last key in the cache after this step
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        if (n_tok[x] > 0) {
            first_pos[x] = p.positions[cu0 + q0 + x * tok_per_tile];
            last_pos[x] = p.positions[cu0 + q0 + x * tok_per_tile + n_tok[x] - 1];
        }
    }
    // query rows: row r of tile x = (token x * tok_per_tile + r / g, head kvh * g + r % g); rows past the portion are zero.
    // Warp 0 takes no part: it starts fetching keys as soon as the barriers exist.  Warp 1 asks for the tensor memory first.
    auto start_queries = [&]() {
        if (warp == 0) return;
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
        }
        const __nv_bfloat16* q_base = p.q + (static_cast<int64_t>(cu0 + q0) * p.H + kvh * g) * HD;
        for (int i = threadIdx.x - 32; i < 2 * kTM * CPR; i += kTcThreads - 32) {
            const int row = i / CPR, c = i % CPR;
            const int x = row >> 7, r = row & 127;
            const int t = row_tok(r), h = r - t * g;
            const bool valid = t < n_tok[x];
            const __nv_bfloat16* src = valid ? q_base + (static_cast<int64_t>(x * tok_per_tile + t) * p.H + h) * HD + c * 8 : p.q;
            cp_async16(reinterpret_cast<__nv_bfloat16*>(sQ + x * L::kTile) + tile_off(r, c), src, valid);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    // Without pieces every block has work: the query rows are on their way while the positions arrive.  With pieces a
    // block first has to know from the positions whether it has any (it asks for nothing it would have to give back).
    if (p.pieces == 1) {
        pdl_wait();
        start_queries();
    }
    // per query tile: the range of key tiles it needs, t_lo <= j < t_hi (none if t_lo >= t_hi)
    int t_lo[2], t_hi[2], key_hi = 0, key_lo = 0x3fffffff;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        if (n_tok[x] > 0) {
            const int first_key = p.window > 0 ? max(0, first_pos[x] - p.window + 1) : 0;   // the oldest key any of its tokens sees
            t_lo[x] = first_key / kTN;
            t_hi[x] = last_pos[x] / kTN + 1;
            key_lo = min(key_lo, first_key);
            key_hi = last_pos[x];                                   // the block's last token
        } else {
            t_lo[x] = 0x3fffffff;
            t_hi[x] = 0;
        }
    }
    int j_lo = min(t_lo[0], t_lo[1]), j_hi = max(t_hi[0], t_hi[1]);
    // A block with many key tiles shares them with up to pieces - 1 other blocks, each at least min_rounds tiles long:
    // piece k of n walks the tiles j_lo + R k / n .. j_lo + R (k + 1) / n of the block's R.  Every piece leaves its
    // unnormalised output, maxima and sums in global memory, and attn_prefill_merge_kernel adds them up and stores the
    // rows.  Blocks beyond n have nothing to do.
    int n_pieces = 1;
    if (p.pieces > 1) {
        const int rounds = j_hi - j_lo;
        n_pieces = min(p.pieces, max(1, rounds / p.min_rounds));
        if (piece >= n_pieces) return;
        if (n_pieces > 1) {
            const int lo = j_lo + (rounds * piece) / n_pieces, hi = j_lo + (rounds * (piece + 1)) / n_pieces;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                t_lo[x] = max(t_lo[x], lo);
                t_hi[x] = min(t_hi[x], hi);
                if (t_lo[x] >= t_hi[x]) { t_lo[x] = 0x3fffffff; t_hi[x] = 0; }
            }
            j_lo = min(t_lo[0], t_lo[1]);
            j_hi = max(t_hi[0], t_hi[1]);
        }
    }
    const int part_slot = (block_id * p.KV + kvh) * p.pieces + piece;
    if (p.pieces > 1 && piece == 0 && threadIdx.x == 0) p.piece_counts[block_id * p.KV + kvh] = n_pieces;
    if (p.pieces > 1) {
        pdl_wait();
        start_queries();
    }
    // Loads are clamped to [key_lo, key_hi], the keys that the block's tokens see: a page below the window may have been
    // given back by its request already (its table entry is -1) and is never looked up; rounding a key down to its box
    // stays inside the page that holds it.

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < kStages; ++i) { mbar_init(kv_full + i, 1); mbar_init(kv_empty + i, 1); }
            for (int i = 0; i < 2; ++i) { mbar_init(s_ready + i, 1); mbar_init(p_ready + i, 128); mbar_init(o_done + i, 1); }
            mbar_fence_init();
        }
        __syncwarp();
        asm volatile("bar.arrive 1, %0;\n" ::"n"(kTcThreads) : "memory");       // the others wait for this below
    } else {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        fence_async_smem();                                         // the tensor core reads what these threads wrote
        tc_before();
        asm volatile("bar.sync 1, %0;\n" ::"n"(kTcThreads) : "memory");
        tc_after();
    }
    const uint32_t tmem = warp == 0 ? 0u : *tmem_slot;
    const uint32_t tS[2] = {tmem, tmem + 128};
    const uint32_t tO[2] = {tmem + 256, tmem + 256 + HD};

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n" ::);
    if (warp == 0) {
        // ---- producer: one lane per TMA box (page or 64 keys, times 64-column half, times K and V), so that the
        // block-table reads of a tile are in flight together instead of one after the other ----
        // page size and box rows are powers of two: shifts and masks instead of divisions
        const int box_shift = 31 - __clz(p.box_rows), page_shift = 31 - __clz(p.page_size);
        const int per_tile_shift = (7 - box_shift) + (HD == 128 ? 1 : 0);          // boxes of a tile times 64-column halves
        const int which = lane >> per_tile_shift;    // 0: K, 1: V, above: idle lanes
        const int box = (lane & ((1 << per_tile_shift) - 1)) / (HD / 64), half = lane % (HD / 64);
        // Load i (0 .. n) brings the keys of tile j_lo + i and the values of tile j_lo + i - 1: what step j_lo + i - 1 of
        // the tensor core reads (its PV and the S of the next tile), so one barrier covers a step.
        const int n = j_hi - j_lo;
        for (int i = 0; i <= n; ++i) {
            const int st = i % kStages;
            const bool has = which == 0 ? i < n : (which == 1 && i >= 1);
            int row = 0;
            if (has) {
                const int j = j_lo + i - which;
                int key = min(max(j * kTN + box * p.box_rows, key_lo), key_hi);      // outside the range: the nearest key inside it
                key &= ~(p.box_rows - 1);
                const int slot = key >> page_shift;
                int page = slot < p.table_width ? table[slot] : -1;
                if (page < 0 || page >= p.num_pages) { atomicExch(p.err, 4); page = 0; }
                row = (((page * 2 + which) * p.KV + kvh) << page_shift) + (key & (p.page_size - 1));
            }
            if (lane == 0) {
                if (i >= kStages) mbar_wait(kv_empty + st, ((i / kStages) - 1) & 1, p.err);
                mbar_expect_tx(kv_full + st, L::kTile * ((i < n ? 1 : 0) + (i >= 1 ? 1 : 0)));
            }
            __syncwarp();
            if (has) tma_load_2d(sKV + (2 * st + which) * L::kTile + half * 16384 + box * p.box_rows * 128, &kv_map, kv_full + st, half * 64, row);
        }
    } else if (warp == 1) {
        if (lane == 0) {                             // ---- tensor-core issue ----
            constexpr uint32_t idesc_s = idesc_bf16(kTM, kTN, false);
            constexpr uint32_t idesc_pv = idesc_bf16(kTM, HD, true);
            auto active = [&](int x, int j) { return j >= t_lo[x] && j < t_hi[x]; };
            auto issue_s = [&](int x, int j) {       // S_j(X); the stage with K_j has been waited for
                const int st = (j - j_lo) % kStages;
                const uint32_t q_addr = smem_u32(sQ + x * L::kTile), k_addr = smem_u32(sKV + 2 * st * L::kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
                    umma(tS[x], desc_sw128(q_addr + off, 16, 1024), desc_sw128(k_addr + off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
                }
                tc_commit(s_ready + x);
            };
            mbar_wait(kv_full + 0, 0, p.err);        // the bytes came through the async proxy: the wait itself orders them
#pragma unroll
            for (int x = 0; x < 2; ++x)
                if (active(x, j_lo)) issue_s(x, j_lo);
            tc_commit(kv_empty + 0);
            for (int j = j_lo; j < j_hi; ++j) {
                const int i = j - j_lo + 1, st = i % kStages;                  // load i: V_j and K_{j+1}
                mbar_wait(kv_full + st, (i / kStages) & 1, p.err);
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (!active(x, j)) {
                        // a tile that starts later (window): its first S belongs to the round before its first PV
                        if (j + 1 < j_hi && active(x, j + 1)) issue_s(x, j + 1);
                        continue;
                    }
                    mbar_wait(p_ready + x, (j - t_lo[x]) & 1, p.err);
                    tc_after();
                    const uint32_t v_addr = smem_u32(sKV + (2 * st + 1) * L::kTile);
#pragma unroll
                    for (int k = 0; k < kTN / 16; ++k)   // P: 16 keys = 8 columns of packed pairs; V: 16 keys further down
                        umma_ts(tO[x], tS[x] + k * 8, desc_sw128(v_addr + k * 16 * 128, 16384, 1024), idesc_pv,
                                (j > t_lo[x] || k > 0) ? 1u : 0u);
                    if (active(x, j + 1)) issue_s(x, j + 1);
                    else tc_commit(o_done + x);
                }
                tc_commit(kv_empty + st);
            }
        }
    }
    } else {                                         // ---- softmax: one thread per query row ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;\n" ::);
        const int x = (warp - 4) >> 2;               // query tile
        const int quarter = warp & 3;                // the 32 lanes of tensor memory this warp may touch
        const int r = quarter * 32 + lane;           // row within the tile
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const bool has_keys = t_lo[x] < t_hi[x];
        float m_ref = -INFINITY, l = 0.f;
        if (has_keys) {
            const int r_tok = row_tok(r);
            const int tok_in_tile = min(r_tok, n_tok[x] - 1);
            const int tok = x * tok_per_tile + tok_in_tile;
            const int row_pos = p.positions[cu0 + q0 + tok];
            const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
            for (int j = t_lo[x]; j < t_hi[x]; ++j) {
                const int i = j - t_lo[x];
                const int key0 = j * kTN;
                mbar_wait(s_ready + x, i & 1, p.err);
                tc_after();
                uint32_t v[128];
#pragma unroll
                for (int c = 0; c < 4; ++c) tm_load32(tS[x] + lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
                tm_wait_ld();
                if (key0 + 127 > row_pos) {                                    // keys after the row's own: -inf
                    const int n_keep = row_pos - key0 + 1;
#pragma unroll
                    for (int c = 0; c < 128; ++c) v[c] = c < n_keep ? v[c] : 0xff800000u;
                }
                if (key0 < row_lo) {                                           // keys before the row's window
                    const int n_drop = row_lo - key0;
#pragma unroll
                    for (int c = 0; c < 128; ++c) v[c] = c < n_drop ? 0xff800000u : v[c];
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains of three-input maxima
#pragma unroll
                for (int c = 0; c < 128; c += 8) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) mx[k] = max3(mx[k], __uint_as_float(v[c + 2 * k]), __uint_as_float(v[c + 2 * k + 1]));
                }
                const float m_new = fmaxf(m_ref, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2);
                // the reference maximum follows only when some row of the warp has outgrown it
                const bool grow = m_new > m_ref + kRescaleStep;
                if (__any_sync(0xffffffffu, grow)) {
                    const float m_use = m_new == -INFINITY ? 0.f : m_new;
                    const float factor = ex2(m_ref - m_use);             // 2^(-inf) = 0 before the first key
                    m_ref = m_new;
                    l *= factor;
                    if (i > 0) {                                          // O(X) holds PV_0 .. PV_{j-1}, all done
#pragma unroll
                        for (int c = 0; c < HD; c += 32) {
                            uint32_t o[32];
                            tm_load32(tO[x] + lane_base + c, o);
                            tm_wait_ld();
#pragma unroll
                            for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * factor);
                            tm_store32(tO[x] + lane_base + c, o);
                        }
                    }
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(-m_use, -m_use);
                float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t packed[32];
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        const int c = h * 64 + 2 * k;
                        const float2 arg = __ffma2_rn(make_float2(__uint_as_float(v[c]), __uint_as_float(v[c + 1])), scale2, neg_m2);
                        const float2 pr = make_float2(ex2(arg.x), ex2(arg.y));
                        sum2[k & 1] = __fadd2_rn(sum2[k & 1], pr);
                        __nv_bfloat162 hh = __floats2bfloat162_rn(pr.x, pr.y);
                        packed[k] = *reinterpret_cast<uint32_t*>(&hh);
                    }
                    tm_store32(tS[x] + lane_base + h * 32, packed);     // P over the first 64 columns of S
                }
                l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
                if (key0 + kTN - 1 > seq_last) {
                    // Keys behind the request's last one came along with its last page.  Their probability is 0, but
                    // what a former holder of the page left there (an Inf, a NaN) times 0 would be NaN: thread r clears
                    // row r of the value tile, which load j - j_lo + 1 brought, before the product P V may start.  (The
                    // threads of the other query tile may do the same; they write the same zeros.)
                    const int load = j - j_lo + 1, vst = load % kStages;
                    mbar_wait(kv_full + vst, (load / kStages) & 1, p.err);
                    if (key0 + r > seq_last) {
                        __nv_bfloat16* v_rows = reinterpret_cast<__nv_bfloat16*>(sKV + (2 * vst + 1) * L::kTile);
#pragma unroll
                        for (int c = 0; c < CPR; ++c) *reinterpret_cast<uint4*>(v_rows + tile_off(r, c)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    fence_async_smem();                                       // the tensor core reads through the async proxy
                }
                tm_wait_st();
                tc_before();
                mbar_arrive(p_ready + x);
            }
            mbar_wait(o_done + x, 0, p.err);
            tc_after();
        }
        // The rows go through shared memory (over the query tile, which no product reads any more, in its swizzled
        // layout) so that the stores to global memory are whole rows side by side: a thread that stored its own row
        // would touch 32 lines with every instruction.
        __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(sQ + x * L::kTile);
        auto stage_chunk = [&](int c0, const uint32_t (&o)[32], float inv) {   // 32 columns of the thread's row
#pragma unroll
            for (int k = 0; k < 32; k += 8) {
                uint4 t;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    h[e] = __floats2bfloat162_rn(__uint_as_float(o[k + 2 * e]) * inv, __uint_as_float(o[k + 2 * e + 1]) * inv);
                *reinterpret_cast<uint4*>(stage + tile_off(r, (c0 + k) >> 3)) = t;
            }
        };
        const bool store = has_keys && n_pieces == 1;
        if (store) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tm_load32(tO[x] + lane_base + c0, o);
                tm_wait_ld();
                stage_chunk(c0, o, inv);
            }
        } else if (n_pieces > 1) {
            // ---- one of several pieces: leave its share (unnormalised rows, reference maxima, sums) for
            // attn_prefill_merge_kernel; rows lie side by side so that the threads of a warp write whole lines ----
            float* mine = p.part_o + (static_cast<int64_t>(part_slot) * 2 + x) * (HD * 128) + r;
            float* mine_ml = p.part_ml + (static_cast<int64_t>(part_slot) * 2 + x) * 256 + r;
            if (has_keys) {
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t o[32];
                    tm_load32(tO[x] + lane_base + c0, o);
                    tm_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) __stcg(mine + (c0 + c) * 128, __uint_as_float(o[c]));
                }
            }
            __stcg(mine_ml, has_keys ? m_ref : -INFINITY);
            __stcg(mine_ml + 128, has_keys ? l : 0.f);          // no sum: the piece had no key for this row
        }
        if (store) {
            asm volatile("bar.sync %0, 128;\n" ::"r"(2 + x) : "memory");       // the 128 threads of this query tile
            __nv_bfloat16* out_base = p.out + ((static_cast<int64_t>(cu0 + q0) + x * tok_per_tile) * p.H + kvh * g) * HD;
            // thread r takes chunk r % CPR of the rows r / CPR + k * (128 / CPR): a row's chunks lie in neighbouring lanes
            constexpr int kRowsPerPass = kTM / CPR;
            const int c = r % CPR;
            uint4 held[CPR];
#pragma unroll
            for (int k = 0; k < CPR; ++k) held[k] = *reinterpret_cast<const uint4*>(stage + tile_off(r / CPR + k * kRowsPerPass, c));
#pragma unroll
            for (int k = 0; k < CPR; ++k) {
                const int row = r / CPR + k * kRowsPerPass;
                const int t = row_tok(row), h = row - t * g;
                if (t < n_tok[x]) *reinterpret_cast<uint4*>(out_base + (static_cast<int64_t>(t) * p.H + h) * HD + c * 8) = held[k];
            }
        }
    }
    tc_before();
    __syncthreads();
    if (warp == 1) {
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512));
    }
}

// Adds up the shares of query blocks that attn_prefill_tcgen05_kernel cut into pieces and stores their rows.  Grid:
// (query block * kv head, query tile, 32 columns of the head); thread r owns row r of the query tile.  Piece k weighs
// 2^(its reference maximum - the largest of them); shares are added in the order of the pieces.
__global__ void __launch_bounds__(128)
attn_prefill_merge_kernel(const TcAttnParams p, const int skip_single, const int hd) {
    constexpr int kMaxPieces = 8;
    constexpr int kRowBytes = 64 + 16;                              // 32 bf16 of a row, padded against bank conflicts
    __shared__ __align__(16) unsigned char stage[128 * kRowBytes];
    pdl_trigger();
    const int g = p.H / p.KV;
    const int tok_per_tile = kTM / g, tok_per_block = 2 * tok_per_tile;
    const int block_id = blockIdx.x / p.KV, kvh = blockIdx.x - block_id * p.KV;
    const int x = blockIdx.y, c0 = blockIdx.z * 32, r = threadIdx.x, lane = threadIdx.x & 31;
    int seq = -1, q0 = 0, q_len = 0, cu0 = 0;
    {
        // Which request the query block belongs to: the lanes of a warp take a request each (every warp does the same),
        // count its query blocks, add them up with shuffles and see whose range holds block_id: one trip to memory
        // for up to 32 requests instead of one per request.
        int before = 0;
        for (int s0 = 0; s0 < p.S && seq < 0; s0 += 32) {
            const int s = s0 + lane;
            int a = 0, n = 0;
            if (s < p.S) { a = p.cu_seqlens[s]; n = p.cu_seqlens[s + 1] - a; }
            const int tiles = (s < p.S && !(skip_single && n == 1)) ? (n + tok_per_block - 1) / tok_per_block : 0;
            int upto = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, upto, o);
                if (lane >= o) upto += v;
            }
            const int first = before + upto - tiles;
            const unsigned hit = __ballot_sync(0xffffffffu, tiles > 0 && block_id >= first && block_id < first + tiles);
            if (hit) {
                const int src = __ffs(hit) - 1;
                seq = s0 + src;
                q0 = (block_id - __shfl_sync(0xffffffffu, first, src)) * tok_per_block;
                q_len = __shfl_sync(0xffffffffu, n, src);
                cu0 = __shfl_sync(0xffffffffu, a, src);
            }
            before += __shfl_sync(0xffffffffu, upto, 31);
        }
    }
    if (seq < 0) return;
    const int n_tok = max(0, min(tok_per_tile, q_len - q0 - x * tok_per_tile));
    if (n_tok == 0) return;
    pdl_wait();
    const int n_pieces = min(p.piece_counts[blockIdx.x], kMaxPieces);
    if (n_pieces <= 1) return;                                      // the block stored its rows itself
    const int64_t first = static_cast<int64_t>(blockIdx.x) * p.pieces;
    float w[kMaxPieces], sum[kMaxPieces];
#pragma unroll
    for (int k = 0; k < kMaxPieces; ++k) {
        const float* ml = p.part_ml + ((first + k) * 2 + x) * 256 + r;
        w[k] = k < n_pieces ? __ldcg(ml) : -INFINITY;
        sum[k] = k < n_pieces ? __ldcg(ml + 128) : 0.f;
    }
    float m_all = -INFINITY, l = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPieces; ++k) {
        if (!(sum[k] > 0.f)) w[k] = -INFINITY;                      // a piece without a key for this row
        m_all = fmaxf(m_all, w[k]);
    }
#pragma unroll
    for (int k = 0; k < kMaxPieces; ++k) {
        w[k] = w[k] == -INFINITY ? 0.f : ex2(w[k] - m_all);
        l = __fadd_rn(l, __fmul_rn(sum[k], w[k]));
    }
    float acc[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) acc[c] = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPieces; ++k) {
        if (k >= n_pieces || w[k] == 0.f) continue;
        const float* share = p.part_o + ((first + k) * 2 + x) * (static_cast<int64_t>(hd) * 128) + static_cast<int64_t>(c0) * 128 + r;
#pragma unroll
        for (int c = 0; c < 32; ++c) acc[c] = __fadd_rn(acc[c], __fmul_rn(__ldcg(share + c * 128), w[k]));
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        uint4 t;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(acc[k + 2 * e] * inv, acc[k + 2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(stage + r * kRowBytes + k * 2) = t;
    }
    __syncthreads();
    // four threads store the 64 bytes of a row
    __nv_bfloat16* out_base = p.out + ((static_cast<int64_t>(cu0 + q0) + x * tok_per_tile) * p.H + kvh * g) * hd + c0;
    const int chunk = r & 3;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int row = pass * 32 + (r >> 2);
        const int t = row / g, h = row - t * g;
        if (t < n_tok)
            *reinterpret_cast<uint4*>(out_base + (static_cast<int64_t>(t) * p.H + h) * hd + chunk * 8) =
                *reinterpret_cast<const uint4*>(stage + row * kRowBytes + chunk * 16);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------

static int kv_map_for(CUtensorMap* out, const void* cache, int64_t rows, int hd, int box_rows) {
    return cached_bf16_map(out, cache, rows, hd, 64, box_rows);
}

}  // namespace cvb

using namespace cvb;

// Floats of scratch that `pieces` > 1 needs for num_tiles query blocks: outputs, maxima and sums of every piece.
extern "C" int64_t cvb_attn_prefill_tcgen05_scratch_floats(int num_tiles, int KV, int hd, int pieces) {
    return static_cast<int64_t>(num_tiles) * KV * pieces * 2 * (hd + 2) * 128;
}

// Blocks the grid needs: per request with more than one token, ceil(tokens / (256 / group)) query blocks, times
// `pieces`.  With pieces > 1 a query block whose tokens see at least 2 * min_rounds key tiles of 128 is worked on by up
// to `pieces` blocks of the grid, each with at least min_rounds tiles; `scratch` then holds
// cvb_attn_prefill_tcgen05_scratch_floats floats and `piece_counts` num_tiles * KV ints (both are written before they
// are read), and a second kernel adds the pieces' shares up.
extern "C" int cvb_attn_prefill_tcgen05(void* out, const void* q, const void* cache, const int* block_tables,
                                           int table_width, const int* cu_seqlens, const int* positions, int S,
                                           int num_tiles, int H, int KV, int hd, int page_size, int window, float scale,
                                           int num_pages, int skip_single, int pieces, int min_rounds, float* scratch,
                                           int64_t scratch_floats, int* piece_counts, int* err_flag, cudaStream_t stream) {
    if (num_tiles == 0) return CVB_OK;
    if (num_tiles < 0 || S <= 0 || H <= 0 || KV <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (H % KV) return CVB_E_SHAPE;
    if (hd != 64 && hd != 128) return CVB_E_UNSUPPORTED;
    const int g = H / KV;
    if (g > 16) return CVB_E_UNSUPPORTED;
    if (page_size < 16 || (page_size & (page_size - 1)) != 0) return CVB_E_UNSUPPORTED;
    if (static_cast<int64_t>(num_pages) * 2 * KV * page_size > 2147483647LL) return CVB_E_SIZE;
    if (pieces < 1 || pieces > 8 || min_rounds < 1) return CVB_E_SIZE;     // the kernel adds up at most eight shares
    if (static_cast<int64_t>(num_tiles) * pieces > 2147483647LL) return CVB_E_SIZE;
    if (pieces > 1 && (!scratch || !piece_counts || scratch_floats < cvb_attn_prefill_tcgen05_scratch_floats(num_tiles, KV, hd, pieces)))
        return CVB_E_SCRATCH;
    TcAttnParams p{};
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2eF; p.err = err_flag;
    p.box_rows = page_size < 64 ? page_size : 64;
    p.pieces = pieces; p.min_rounds = min_rounds; p.piece_counts = piece_counts;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + static_cast<int64_t>(num_tiles) * KV * pieces * 2 * hd * 128 : nullptr;
    CUtensorMap map;
    const int rc = kv_map_for(&map, cache, static_cast<int64_t>(num_pages) * 2 * KV * page_size, hd, p.box_rows);
    if (rc != CVB_OK) return rc;
    if (num_tiles > 65535) return CVB_E_SIZE;
    dim3 grid(static_cast<unsigned>(KV), static_cast<unsigned>(num_tiles), static_cast<unsigned>(pieces));
    if (hd == 128) {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem<128>::kBytes); set = true; }
        launch_kernel(attn_prefill_tcgen05_kernel<128>, grid, dim3(kTcThreads), TcSmem<128>::kBytes, stream, map, p, skip_single);
    } else {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem<64>::kBytes); set = true; }
        launch_kernel(attn_prefill_tcgen05_kernel<64>, grid, dim3(kTcThreads), TcSmem<64>::kBytes, stream, map, p, skip_single);
    }
    const int launched = launch_status();
    if (launched != CVB_OK || pieces == 1) return launched;
    if (static_cast<int64_t>(num_tiles) * KV > 2147483647LL) return CVB_E_SIZE;
    launch_kernel(attn_prefill_merge_kernel, dim3(static_cast<unsigned>(num_tiles * KV), 2, static_cast<unsigned>(hd / 32)), dim3(128), 0,
                  stream, p, skip_single, hd);
    return launch_status();
}
