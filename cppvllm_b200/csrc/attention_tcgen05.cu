// Flash attention for prompt portions on the fifth-generation tensor cores (tcgen05), bf16, head sizes 64 and 128,
// over the paged cache with a causal offset (and an optional window).  Same arithmetic as attention_bf16.cu (reference
// kernels/paged_attention.cu:89-359: scale * q.k over keys lo..p, online softmax in float, o = sum p v / l).
//
// One block owns 128 query rows of one kv head: the query heads that share the kv head are packed next to each other
// (row r = token r / g, head kvh * g + r % g), so a key/value tile is fetched once for the whole group.  Keys are
// walked in tiles of 128.  Roles, by warp:
//   warp 0     producer: one thread issues TMA copies (one box per page and 64-column half, 128-byte swizzle) of K tiles
//              into a ring of three stages and of V tiles into a ring of two;
//   warp 1     allocates 512 columns of tensor memory; one thread issues the products
//                  S_j  = Q K_j^T   (M 128, N 128, K = head size; both operands K-major)       -> S buffer j % 2
//                  PV_j = P_j V_j   (M 128, N = head size, K 128; P K-major, V MN-major)      -> PV buffer j % 2
//              in the order S_0, S_1, PV_0, S_2, PV_1, ... so that the softmax of tile j + 1 runs beside PV_j;
//   warps 2-9  softmax: two threads per query row, one for keys 0..63 of the tile and one for keys 64..127 (and the same
//              halves of the output row).  A thread reads its half row of S_j with tcgen05.ld once, takes the
//              maximum, swaps it with its partner through shared memory (one named barrier per tile), writes its half
//              of P_j as bf16 into shared memory in the layout the tensor core reads, and then adds its half of
//              PV_{j-1} from tensor memory into its float accumulator (rescaled by the change of the maximum).
// Buffers are handed over with mbarriers: TMA transaction counts, tcgen05.commit arrivals from the tensor core, and
// plain arrivals from the 256 softmax threads.  Every wait is bounded by a cycle count; a wait that runs out records
// error 5 and the block runs on to its end (tensor memory is always given back).
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace cvb {

constexpr int kTM = 128;                      // query rows per block
constexpr int kTN = 128;                      // keys per tile
constexpr int kKStages = 3;
constexpr int kVStages = 2;
constexpr int kSoftmaxThreads = 256;           // two threads per query row: each owns half of the columns
constexpr int kTcThreads = 64 + kSoftmaxThreads;
constexpr float kLog2eF = 1.4426950408889634f;

__device__ __forceinline__ uint32_t saddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mb_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%1], %0;\n" ::"r"(count), "r"(saddr(bar)));
}
__device__ __forceinline__ void mb_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%1], %0;\n" ::"r"(bytes), "r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void mb_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ bool mb_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred P1;\nmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\nselp.b32 %0, 1, 0, P1;\n}\n"
                 : "=r"(ok) : "r"(saddr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mb_wait(uint64_t* bar, uint32_t parity, int* err) {
    if (mb_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    while (!mb_try_wait(bar, parity)) {
        if (clock64() - t0 > 40000000LL) { atomicExch(err, 5); return; }
    }
}
__device__ __forceinline__ void tma_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(saddr(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(saddr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void cpa16(void* smem, const void* gmem, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(saddr(smem)), "l"(gmem), "r"(n));
}

// Shared-memory matrix descriptors, 128-byte swizzle, rows of 128 bytes in 1024-byte atoms of 8 rows.
//   K-major operand ([rows][64 elements] per half): stride byte offset 1024 between 8-row groups.
//   MN-major operand (V: [keys][64 head elements] per half): the 64 contiguous elements run along N, keys along K;
//   stride byte offset 1024 between groups of 8 keys, leading byte offset = distance between the 64-column halves.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void commit_to(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tm_load32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                   "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                   "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tm_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

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
};

template <int HD>
struct TcSmem {
    static constexpr int kTile = 128 * HD * 2;                       // bytes of a [128][HD] bf16 tile
    static constexpr int kP = 128 * kTN * 2;                         // bytes of P [128][128]
    static constexpr int kNumBars = 2 * kKStages + 2 * kVStages + 2 + 2 + 1 + 1 + 2 + 2;
    // no slack for alignment: with 128-wide heads the tiles leave 3 KB of the 227 KB; the kernel checks the base instead
    static constexpr size_t kBytes = static_cast<size_t>(kTile) * (1 + kKStages + kVStages) + kP + kNumBars * 8 + 16 + 2 * 2 * 128 * 4;
};

// One thread: fetch keys [key0, key0 + 128) of one kv head (`which` 0 = K, 1 = V) into a tile.
template <int HD>
__device__ __forceinline__ void issue_tile(unsigned char* tile, uint64_t* bar, const CUtensorMap* map, const TcAttnParams& p,
                                           const int* table, int kvh, int which, int key0, int key_lo, int key_hi) {
    mb_expect_tx(bar, TcSmem<HD>::kTile);
    for (int b0 = 0; b0 < kTN; b0 += p.box_rows) {
        int key = min(max(key0 + b0, key_lo), key_hi);              // outside the range: the nearest key inside it
        key -= key % p.box_rows;
        const int slot = key / p.page_size;
        int page = slot < p.table_width ? table[slot] : -1;
        if (page < 0 || page >= p.num_pages) { atomicExch(p.err, 4); page = 0; }
        const int row = ((page * 2 + which) * p.KV + kvh) * p.page_size + key % p.page_size;
#pragma unroll
        for (int half = 0; half < HD / 64; ++half)
            tma_2d(tile + half * 16384 + b0 * 128, map, bar, half * 64, row);
    }
}

template <int HD>
__global__ void __launch_bounds__(kTcThreads)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap kv_map, const TcAttnParams p, const int skip_single) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using L = TcSmem<HD>;
    pdl_trigger();
    if ((saddr(smem_raw) & 1023u) != 0) {            // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicExch(p.err, 6);
        return;
    }
    unsigned char* sQ = smem_raw;
    unsigned char* sK = sQ + L::kTile;
    unsigned char* sV = sK + kKStages * L::kTile;
    unsigned char* sP = sV + kVStages * L::kTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + L::kP);
    uint64_t* k_full = bars;                       // [3]  TMA
    uint64_t* k_empty = k_full + kKStages;         // [3]  tensor core
    uint64_t* v_full = k_empty + kKStages;         // [2]  TMA
    uint64_t* v_empty = v_full + kVStages;         // [2]  tensor core
    uint64_t* s_full = v_empty + kVStages;         // [2]  tensor core
    uint64_t* s_empty = s_full + 2;                // [2]  128 softmax threads
    uint64_t* p_full = s_empty + 2;                // [1]  128 softmax threads
    uint64_t* p_empty = p_full + 1;                // [1]  tensor core
    uint64_t* pv_full = p_empty + 1;               // [2]  tensor core
    uint64_t* pv_empty = pv_full + 2;              // [2]  128 softmax threads
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_empty + 2);
    float* xch = reinterpret_cast<float*>(tmem_slot + 4);           // [2 tiles in flight][2 halves][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = p.H / p.KV;
    const int tok_per_tile = kTM / g;
    const int kvh = blockIdx.y;
    constexpr int CPR = HD / 8;

    // which request and which tile of it; long tiles (late in the request) come first in the grid
    int seq = -1, q0 = 0, q_len = 0, cu0 = 0;
    {
        int tile = gridDim.x - 1 - blockIdx.x;
        for (int s = 0; s < p.S; ++s) {
            const int a = p.cu_seqlens[s], n = p.cu_seqlens[s + 1] - a;
            if (skip_single && n == 1) continue;
            const int tiles = (n + tok_per_tile - 1) / tok_per_tile;
            if (tile < tiles) { seq = s; q0 = tile * tok_per_tile; q_len = n; cu0 = a; break; }
            tile -= tiles;
        }
    }
    if (seq < 0) return;
    pdl_wait();
    const int n_tok = min(tok_per_tile, q_len - q0);
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    const int pos_first = p.positions[cu0 + q0];
    const int pos_last = p.positions[cu0 + q0 + n_tok - 1];
    const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int key_hi = pos_last;
    const int tile_begin = key_lo / kTN, n_tiles = key_hi / kTN - tile_begin + 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kKStages; ++i) { mb_init(k_full + i, 1); mb_init(k_empty + i, 1); }
        for (int i = 0; i < kVStages; ++i) { mb_init(v_full + i, 1); mb_init(v_empty + i, 1); }
        for (int i = 0; i < 2; ++i) {
            mb_init(s_full + i, 1); mb_init(s_empty + i, kSoftmaxThreads);
            mb_init(pv_full + i, 1); mb_init(pv_empty + i, kSoftmaxThreads);
        }
        mb_init(p_full, kSoftmaxThreads);
        mb_init(p_empty, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // the query tile: row r = (token r / g, head kvh * g + r % g); rows past the portion are zero
    for (int i = threadIdx.x; i < kTM * CPR; i += kTcThreads) {
        const int r = i / CPR, c = i % CPR;
        const int tok = r / g;
        const bool valid = tok < n_tok;
        const __nv_bfloat16* src = valid ? p.q + ((static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * HD + c * 8) : p.q;
        cpa16(reinterpret_cast<__nv_bfloat16*>(sQ) + tile_off(r, c), src, valid);
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
    fence_async_smem();                              // the tensor core reads what these threads wrote
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS[2] = {tmem, tmem + 128};
    const uint32_t tPV[2] = {tmem + 256, tmem + 256 + HD};

    if (warp == 0) {
        if (lane == 0) {                             // ---- producer ----
            for (int j = 0; j < n_tiles; ++j) {
                const int ks = j % kKStages, vs = j % kVStages;
                if (j >= kKStages) mb_wait(k_empty + ks, ((j / kKStages) - 1) & 1, p.err);
                issue_tile<HD>(sK + ks * L::kTile, k_full + ks, &kv_map, p, table, kvh, 0, (tile_begin + j) * kTN, key_lo, key_hi);
                if (j >= kVStages) mb_wait(v_empty + vs, ((j / kVStages) - 1) & 1, p.err);
                issue_tile<HD>(sV + vs * L::kTile, v_full + vs, &kv_map, p, table, kvh, 1, (tile_begin + j) * kTN, key_lo, key_hi);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                             // ---- tensor-core issue ----
            constexpr uint32_t idesc_s = idesc_bf16(kTM, kTN, false);
            constexpr uint32_t idesc_pv = idesc_bf16(kTM, HD, true);
            const uint32_t q_addr = saddr(sQ), p_addr = saddr(sP);
            auto issue_s = [&](int j) {
                const int ks = j % kKStages, b = j & 1;
                mb_wait(k_full + ks, (j / kKStages) & 1, p.err);
                if (j >= 2) mb_wait(s_empty + b, ((j >> 1) - 1) & 1, p.err);
                tc_after();
                const uint32_t k_addr = saddr(sK + ks * L::kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;         // half, then 32 bytes per k-step
                    umma(tS[b], desc_sw128(q_addr + off, 16, 1024), desc_sw128(k_addr + off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
                }
                commit_to(s_full + b);
                commit_to(k_empty + ks);
            };
            issue_s(0);
            for (int j = 0; j < n_tiles; ++j) {
                if (j + 1 < n_tiles) issue_s(j + 1);
                const int vs = j % kVStages, b = j & 1;
                mb_wait(v_full + vs, (j / kVStages) & 1, p.err);
                mb_wait(p_full, j & 1, p.err);
                if (j >= 2) mb_wait(pv_empty + b, ((j >> 1) - 1) & 1, p.err);
                tc_after();
                const uint32_t v_addr = saddr(sV + vs * L::kTile);
#pragma unroll
                for (int k = 0; k < kTN / 16; ++k) {
                    const uint32_t a_off = (k >> 2) * 16384 + (k & 3) * 32;       // P: K-major, keys along K
                    const uint32_t b_off = k * 16 * 128;                          // V: 16 keys further down
                    umma(tPV[b], desc_sw128(p_addr + a_off, 16, 1024), desc_sw128(v_addr + b_off, 16384, 1024), idesc_pv, k > 0 ? 1u : 0u);
                }
                commit_to(pv_full + b);
                commit_to(p_empty);
                commit_to(v_empty + vs);
            }
        }
    } else {                                         // ---- softmax: two threads per query row ----
        constexpr int HC = HD / 2;                   // output columns per thread
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;            // 0: keys / columns of the first half, 1: of the second
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const int tok = min(r / g, n_tok - 1);
        const int row_pos = p.positions[cu0 + q0 + tok];
        const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
        float o[HC];
#pragma unroll
        for (int i = 0; i < HC; ++i) o[i] = 0.f;
        float m = -INFINITY, l = 0.f, corr_prev = 0.f;
        __nv_bfloat16* prow = reinterpret_cast<__nv_bfloat16*>(sP);

        auto add_pv = [&](int j, float corr) {      // o = o * corr + (this thread's half of) PV_j
            const int b = j & 1;
            mb_wait(pv_full + b, (j >> 1) & 1, p.err);
            tc_after();
            const float2 corr2 = make_float2(corr, corr);
#pragma unroll
            for (int c0 = 0; c0 < HC; c0 += 32) {
                uint32_t v[32];
                tm_load32(tPV[b] + lane_base + half * HC + c0, v);
                tm_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {                    // two columns per packed multiply-add
                    const float2 acc = __ffma2_rn(make_float2(o[c0 + i], o[c0 + i + 1]), corr2,
                                                  make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
                    o[c0 + i] = acc.x;
                    o[c0 + i + 1] = acc.y;
                }
            }
            tc_before();
            mb_arrive(pv_empty + b);
        };

        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            const int key0 = (tile_begin + j) * kTN + half * 64;     // first key of this thread's 64
            const bool need_mask = key0 + 63 > row_pos || key0 < row_lo;
            mb_wait(s_full + b, (j >> 1) & 1, p.err);
            tc_after();
            uint32_t v[64];
            tm_load32(tS[b] + lane_base + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
            tm_load32(tS[b] + lane_base + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
            tm_wait_ld();
            tc_before();
            mb_arrive(s_empty + b);                                  // S_j is in registers: its buffer may be refilled
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = key0 + i;
                    if (key > row_pos || key < row_lo) v[i] = 0xff800000u;     // -inf
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains instead of one long one
#pragma unroll
            for (int i = 0; i < 64; i += 4) {
#pragma unroll
                for (int k = 0; k < 4; ++k) mx[k] = fmaxf(mx[k], __uint_as_float(v[i + k]));
            }
            float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            // the row's maximum is the larger of the two halves'
            xch[(b * 2 + half) * 128 + r] = tile_max;
            asm volatile("bar.sync 1, %0;\n" ::"n"(kSoftmaxThreads) : "memory");
            tile_max = fmaxf(tile_max, xch[(b * 2 + (half ^ 1)) * 128 + r]);
            const float m_new = fmaxf(m, tile_max * p.scale_log2);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = ex2(m - m_use);                       // 2^(-inf) = 0 at the first tile
            m = m_new;
            // probabilities, rounded to bf16, into this thread's half row of the P tile (free once PV_{j-1} has read it)
            if (j > 0) mb_wait(p_empty, (j - 1) & 1, p.err);
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg_m2 = make_float2(-m_use, -m_use);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 arg = __ffma2_rn(make_float2(__uint_as_float(v[c * 8 + 2 * i]), __uint_as_float(v[c * 8 + 2 * i + 1])),
                                                  scale2, neg_m2);
                    const float2 pr = make_float2(ex2(arg.x), ex2(arg.y));
                    sum2[i & 1] = __fadd2_rn(sum2[i & 1], pr);
                    __nv_bfloat162 h = __floats2bfloat162_rn(pr.x, pr.y);
                    packed[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(prow + tile_off(r, half * 8 + c)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            const float tile_sum = (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
            l = l * corr + tile_sum;
            fence_async_smem();                                      // P_j is visible to the tensor core
            mb_arrive(p_full);
            if (j > 0) add_pv(j - 1, corr_prev);
            corr_prev = corr;
        }
        add_pv(n_tiles - 1, corr_prev);

        // the row's sum is the sum of the two halves'
        asm volatile("bar.sync 1, %0;\n" ::"n"(kSoftmaxThreads) : "memory");      // everyone has read the last maxima
        xch[half * 128 + r] = l;
        asm volatile("bar.sync 1, %0;\n" ::"n"(kSoftmaxThreads) : "memory");
        l += xch[(half ^ 1) * 128 + r];
        if (r / g < n_tok) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.out + (static_cast<int64_t>(cu0 + q0 + r / g) * p.H + kvh * g + r % g) * HD + half * HC;
#pragma unroll
            for (int c = 0; c < HC; c += 8) {
                uint4 t;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(o[c + 2 * i] * inv, o[c + 2 * i + 1] * inv);
                *reinterpret_cast<uint4*>(dst + c) = t;
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

// ---- two query tiles per block -------------------------------------------------------------------------------------
// One block owns 256 query rows of one kv head as two tiles X = A, B of 128 rows, and the tensor core alternates between
// them: while the softmax of one tile runs, the products of the other do.
//   warp 0     producer (TMA), K ring of three stages, V ring of two; a K/V tile serves both query tiles;
//   warp 1     one thread issues, per key tile j and query tile X:  PV_j(X) = P_j(X) V_j  accumulated into O(X) in tensor
//              memory, then S_{j+1}(X) = Q(X) K_{j+1}^T.  P_j(X) is read from tensor memory, where the softmax threads put
//              it over the first half of S_j(X);
//   warps 4-7  softmax of tile A, warps 8-11 of tile B: one thread per query row (registers move from the first warpgroup
//              to these two with setmaxnreg).  A thread reads its row of S (128 floats),
//              exponentiates against a reference maximum, writes the row of P as bf16 back into tensor memory.  The output
//              accumulator stays in tensor memory; it is rescaled (read, multiplied, written back by the row's thread) only
//              when the running maximum of some row of the warp has grown by more than 2^8 since the reference was set,
//              which happens in the first tiles and then hardly ever.  The result is exact: the same reference scales
//              P and the row sum.
// Tensor memory columns: S(A) 0..127, S(B) 128..255, O(A) 256.., O(B) 256 + HD...
constexpr int kPPThreads = 128 + 256;         // one warpgroup of helpers (two warps idle), one warpgroup per query tile

template <int HD>
struct PPSmem {
    static constexpr int kTile = 128 * HD * 2;
    static constexpr int kNumBars = 2 * kKStages + 2 * kVStages + 2 + 2 + 2;
    static constexpr size_t kBytes = static_cast<size_t>(kTile) * (2 + kKStages + kVStages) + kNumBars * 8 + 16;
};

__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tm_store32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                   "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
                   "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
                   "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                 : "memory");
}
__device__ __forceinline__ void tm_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

constexpr float kRescaleStep = 8.f;            // log2 of the growth of a row's maximum that forces a rescale

template <int HD>
__global__ void __launch_bounds__(kPPThreads, 1)
attn_prefill_tcgen05_2q_kernel(const __grid_constant__ CUtensorMap kv_map, const TcAttnParams p, const int skip_single) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using L = PPSmem<HD>;
    pdl_trigger();
    if ((saddr(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(p.err, 6);
        return;
    }
    unsigned char* sQ = smem_raw;                                   // two tiles
    unsigned char* sK = sQ + 2 * L::kTile;
    unsigned char* sV = sK + kKStages * L::kTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kVStages * L::kTile);
    uint64_t* k_full = bars;                       // [3]  TMA
    uint64_t* k_empty = k_full + kKStages;         // [3]  tensor core
    uint64_t* v_full = k_empty + kKStages;         // [2]  TMA
    uint64_t* v_empty = v_full + kVStages;         // [2]  tensor core
    uint64_t* s_ready = v_empty + kVStages;        // [2 tiles]  tensor core: S_j(X) and everything issued before it is done
    uint64_t* p_ready = s_ready + 2;               // [2 tiles]  128 softmax threads: P_j(X) is in tensor memory
    uint64_t* o_done = p_ready + 2;                // [2 tiles]  tensor core: the last PV(X) is done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = p.H / p.KV;
    const int tok_per_tile = kTM / g;
    const int tok_per_block = 2 * tok_per_tile;
    const int kvh = blockIdx.y;
    constexpr int CPR = HD / 8;

    int seq = -1, q0 = 0, q_len = 0, cu0 = 0;
    {
        int tile = gridDim.x - 1 - blockIdx.x;                      // long blocks (late in the request) come first
        for (int s = 0; s < p.S; ++s) {
            const int a = p.cu_seqlens[s], n = p.cu_seqlens[s + 1] - a;
            if (skip_single && n == 1) continue;
            const int tiles = (n + tok_per_block - 1) / tok_per_block;
            if (tile < tiles) { seq = s; q0 = tile * tok_per_block; q_len = n; cu0 = a; break; }
            tile -= tiles;
        }
    }
    if (seq < 0) return;
    pdl_wait();
    const int* table = p.block_tables + static_cast<int64_t>(seq) * p.table_width;
    // per query tile: its tokens, and the range of key tiles it needs
    int n_tok[2], t_lo[2], t_hi[2];                                 // key tiles t_lo <= j < t_hi (none if t_lo >= t_hi)
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        n_tok[x] = max(0, min(tok_per_tile, q_len - q0 - x * tok_per_tile));
        if (n_tok[x] > 0) {
            const int first = p.positions[cu0 + q0 + x * tok_per_tile];
            const int last = p.positions[cu0 + q0 + x * tok_per_tile + n_tok[x] - 1];
            t_lo[x] = (p.window > 0 ? max(0, first - p.window + 1) : 0) / kTN;
            t_hi[x] = last / kTN + 1;
        } else {
            t_lo[x] = 0x3fffffff;
            t_hi[x] = 0;
        }
    }
    const int j_lo = min(t_lo[0], t_lo[1]), j_hi = max(t_hi[0], t_hi[1]);
    const int key_lo = j_lo * kTN;                                  // keys that exist for the clamp of the loads
    const int key_hi = p.positions[cu0 + q0 + n_tok[0] + n_tok[1] - 1];

    if (threadIdx.x == 0) {
        for (int i = 0; i < kKStages; ++i) { mb_init(k_full + i, 1); mb_init(k_empty + i, 1); }
        for (int i = 0; i < kVStages; ++i) { mb_init(v_full + i, 1); mb_init(v_empty + i, 1); }
        for (int i = 0; i < 2; ++i) { mb_init(s_ready + i, 1); mb_init(p_ready + i, 128); mb_init(o_done + i, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(saddr(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // query rows: row r of tile x = (token x * tok_per_tile + r / g, head kvh * g + r % g); rows past the portion are zero
    for (int i = threadIdx.x; i < 2 * kTM * CPR; i += kPPThreads) {
        const int row = i / CPR, c = i % CPR;
        const int x = row >> 7, r = row & 127;
        const int tok = x * tok_per_tile + r / g;
        const bool valid = r / g < n_tok[x];
        const __nv_bfloat16* src = valid ? p.q + ((static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * HD + c * 8) : p.q;
        cpa16(reinterpret_cast<__nv_bfloat16*>(sQ + x * L::kTile) + tile_off(r, c), src, valid);
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
    fence_async_smem();
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS[2] = {tmem, tmem + 128};
    const uint32_t tO[2] = {tmem + 256, tmem + 256 + HD};

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n" ::);
    if (warp == 0) {
        if (lane == 0) {                             // ---- producer ----
            for (int j = j_lo; j < j_hi; ++j) {
                const int i = j - j_lo, ks = i % kKStages, vs = i % kVStages;
                if (i >= kKStages) mb_wait(k_empty + ks, ((i / kKStages) - 1) & 1, p.err);
                issue_tile<HD>(sK + ks * L::kTile, k_full + ks, &kv_map, p, table, kvh, 0, j * kTN, key_lo, key_hi);
                if (i >= kVStages) mb_wait(v_empty + vs, ((i / kVStages) - 1) & 1, p.err);
                issue_tile<HD>(sV + vs * L::kTile, v_full + vs, &kv_map, p, table, kvh, 1, j * kTN, key_lo, key_hi);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                             // ---- tensor-core issue ----
            constexpr uint32_t idesc_s = idesc_bf16(kTM, kTN, false);
            constexpr uint32_t idesc_pv = idesc_bf16(kTM, HD, true);
            auto active = [&](int x, int j) { return j >= t_lo[x] && j < t_hi[x]; };
            auto issue_s = [&](int x, int j) {       // S_j(X); the K tile has been waited for
                const int ks = (j - j_lo) % kKStages;
                const uint32_t q_addr = saddr(sQ + x * L::kTile), k_addr = saddr(sK + ks * L::kTile);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
                    umma(tS[x], desc_sw128(q_addr + off, 16, 1024), desc_sw128(k_addr + off, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
                }
                commit_to(s_ready + x);
            };
            auto wait_k = [&](int j) {
                const int i = j - j_lo;
                mb_wait(k_full + i % kKStages, (i / kKStages) & 1, p.err);
                tc_after();
            };
            {
                wait_k(j_lo);
#pragma unroll
                for (int x = 0; x < 2; ++x)
                    if (active(x, j_lo)) issue_s(x, j_lo);
                commit_to(k_empty + 0);
            }
            for (int j = j_lo; j < j_hi; ++j) {
                const int i = j - j_lo, vs = i % kVStages;
                bool have_v = false, have_k = false;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (!active(x, j)) {
                        // a tile that starts later (window): its first S belongs to the round before its first PV
                        if (j + 1 < j_hi && active(x, j + 1)) {
                            if (!have_k) { wait_k(j + 1); have_k = true; }
                            issue_s(x, j + 1);
                        }
                        continue;
                    }
                    mb_wait(p_ready + x, (j - t_lo[x]) & 1, p.err);
                    if (!have_v) { mb_wait(v_full + vs, (i / kVStages) & 1, p.err); have_v = true; }
                    tc_after();
                    const uint32_t v_addr = saddr(sV + vs * L::kTile);
#pragma unroll
                    for (int k = 0; k < kTN / 16; ++k)   // P: 16 keys = 8 columns of packed pairs; V: 16 keys further down
                        umma_ts(tO[x], tS[x] + k * 8, desc_sw128(v_addr + k * 16 * 128, 16384, 1024), idesc_pv,
                                (j > t_lo[x] || k > 0) ? 1u : 0u);
                    if (active(x, j + 1)) {
                        if (!have_k) { wait_k(j + 1); have_k = true; }
                        issue_s(x, j + 1);
                    } else {
                        commit_to(o_done + x);
                    }
                }
                if (!have_v) mb_wait(v_full + vs, (i / kVStages) & 1, p.err);    // nobody needed it: hand it back in order
                commit_to(v_empty + vs);
                if (j + 1 < j_hi) {
                    if (!have_k) wait_k(j + 1);          // nobody needs it: still hand the stage back in order
                    commit_to(k_empty + (i + 1) % kKStages);
                }
            }
        }
    }
    } else {                                         // ---- softmax: one thread per query row ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;\n" ::);
        const int x = (warp - 4) >> 2;               // query tile
        const int quarter = warp & 3;                // the 32 lanes of tensor memory this warp may touch
        const int r = quarter * 32 + lane;           // row within the tile
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        if (t_lo[x] < t_hi[x]) {
            const int tok_in_tile = min(r / g, n_tok[x] - 1);
            const int tok = x * tok_per_tile + tok_in_tile;
            const int row_pos = p.positions[cu0 + q0 + tok];
            const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
            float m_ref = -INFINITY, l = 0.f;
            for (int j = t_lo[x]; j < t_hi[x]; ++j) {
                const int i = j - t_lo[x];
                const int key0 = j * kTN;
                mb_wait(s_ready + x, i & 1, p.err);
                tc_after();
                uint32_t v[128];
#pragma unroll
                for (int c = 0; c < 4; ++c) tm_load32(tS[x] + lane_base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
                tm_wait_ld();
                if (key0 + 127 > row_pos || key0 < row_lo) {
#pragma unroll
                    for (int c = 0; c < 128; ++c) {
                        const int key = key0 + c;
                        if (key > row_pos || key < row_lo) v[c] = 0xff800000u;     // -inf
                    }
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 128; c += 4) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) mx[k] = fmaxf(mx[k], __uint_as_float(v[c + k]));
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
                tm_wait_st();
                tc_before();
                mb_arrive(p_ready + x);
            }
            mb_wait(o_done + x, 0, p.err);
            tc_after();
            const bool valid = r / g < n_tok[x];
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.out + (static_cast<int64_t>(cu0 + q0 + tok) * p.H + kvh * g + r % g) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t o[32];
                tm_load32(tO[x] + lane_base + c, o);
                tm_wait_ld();
                if (valid) {
#pragma unroll
                    for (int k = 0; k < 32; k += 8) {
                        uint4 t;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            h[e] = __floats2bfloat162_rn(__uint_as_float(o[k + 2 * e]) * inv, __uint_as_float(o[k + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + k) = t;
                    }
                }
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

// ---- host side ------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    });
    return fn;
}

static int kv_map_for(CUtensorMap* out, const void* cache, int64_t rows, int hd, int box_rows) {
    struct Key { const void* p; int64_t rows; int hd, box; bool operator==(const Key& o) const { return p == o.p && rows == o.rows && hd == o.hd && box == o.box; } };
    struct Hash { size_t operator()(const Key& k) const { return std::hash<const void*>()(k.p) ^ (std::hash<int64_t>()(k.rows) * 31) ^ (k.hd * 131) ^ (k.box * 7); } };
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{cache, rows, hd, box_rows};
    auto it = maps.find(key);
    if (it == maps.end()) {
        EncodeFn fn = encode_fn();
        if (fn == nullptr) return CVB_E_UNSUPPORTED;
        if ((reinterpret_cast<uintptr_t>(cache) & 15) != 0) return CVB_E_ALIGN;
        CUtensorMap m;
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(hd), static_cast<cuuint64_t>(rows)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(hd) * sizeof(__nv_bfloat16)};
        const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
        const cuuint32_t estr[2] = {1u, 1u};
        if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return CVB_E_SHAPE;
        it = maps.emplace(key, m).first;
    }
    *out = it->second;
    return CVB_OK;
}

}  // namespace cvb

using namespace cvb;

// Tiles the grid needs: per request with more than one token, ceil(tokens / (128 / group)).
extern "C" int cvb_attn_prefill_tcgen05(void* out, const void* q, const void* cache, const int* block_tables,
                                        int table_width, const int* cu_seqlens, const int* positions, int S,
                                        int num_tiles, int H, int KV, int hd, int page_size, int window, float scale,
                                        int num_pages, int skip_single, int* err_flag, cudaStream_t stream) {
    if (num_tiles == 0) return CVB_OK;
    if (num_tiles < 0 || S <= 0 || H <= 0 || KV <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (H % KV) return CVB_E_SHAPE;
    if (hd != 64 && hd != 128) return CVB_E_UNSUPPORTED;
    if (H / KV > 16 || KV > 65535) return CVB_E_UNSUPPORTED;
    if (page_size < 16 || (page_size & (page_size - 1)) != 0) return CVB_E_UNSUPPORTED;
    if (static_cast<int64_t>(num_pages) * 2 * KV * page_size > 2147483647LL) return CVB_E_SIZE;
    TcAttnParams p{};
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2eF; p.err = err_flag;
    p.box_rows = page_size < 64 ? page_size : 64;
    CUtensorMap map;
    const int rc = kv_map_for(&map, cache, static_cast<int64_t>(num_pages) * 2 * KV * page_size, hd, p.box_rows);
    if (rc != CVB_OK) return rc;
    dim3 grid(static_cast<unsigned>(num_tiles), static_cast<unsigned>(KV));
    if (hd == 128) {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem<128>::kBytes); set = true; }
        launch_kernel(attn_prefill_tcgen05_kernel<128>, grid, dim3(kTcThreads), TcSmem<128>::kBytes, stream, map, p, skip_single);
    } else {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem<64>::kBytes); set = true; }
        launch_kernel(attn_prefill_tcgen05_kernel<64>, grid, dim3(kTcThreads), TcSmem<64>::kBytes, stream, map, p, skip_single);
    }
    return launch_status();
}

// Blocks the grid needs: per request with more than one token, ceil(tokens / (256 / group)).
extern "C" int cvb_attn_prefill_tcgen05_2q(void* out, const void* q, const void* cache, const int* block_tables,
                                           int table_width, const int* cu_seqlens, const int* positions, int S,
                                           int num_tiles, int H, int KV, int hd, int page_size, int window, float scale,
                                           int num_pages, int skip_single, int* err_flag, cudaStream_t stream) {
    if (num_tiles == 0) return CVB_OK;
    if (num_tiles < 0 || S <= 0 || H <= 0 || KV <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0) return CVB_E_SIZE;
    if (H % KV) return CVB_E_SHAPE;
    if (hd != 64 && hd != 128) return CVB_E_UNSUPPORTED;
    const int g = H / KV;
    if (g > 16 || KV > 65535) return CVB_E_UNSUPPORTED;
    if (page_size < 16 || (page_size & (page_size - 1)) != 0) return CVB_E_UNSUPPORTED;
    if (static_cast<int64_t>(num_pages) * 2 * KV * page_size > 2147483647LL) return CVB_E_SIZE;
    TcAttnParams p{};
    p.out = (__nv_bfloat16*)out; p.q = (const __nv_bfloat16*)q;
    p.block_tables = block_tables; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.table_width = table_width; p.S = S; p.H = H; p.KV = KV; p.page_size = page_size; p.window = window;
    p.num_pages = num_pages; p.scale_log2 = scale * kLog2eF; p.err = err_flag;
    p.box_rows = page_size < 64 ? page_size : 64;
    CUtensorMap map;
    const int rc = kv_map_for(&map, cache, static_cast<int64_t>(num_pages) * 2 * KV * page_size, hd, p.box_rows);
    if (rc != CVB_OK) return rc;
    dim3 grid(static_cast<unsigned>(num_tiles), static_cast<unsigned>(KV));
    if (hd == 128) {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_tcgen05_2q_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PPSmem<128>::kBytes); set = true; }
        launch_kernel(attn_prefill_tcgen05_2q_kernel<128>, grid, dim3(kPPThreads), PPSmem<128>::kBytes, stream, map, p, skip_single);
    } else {
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(attn_prefill_tcgen05_2q_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PPSmem<64>::kBytes); set = true; }
        launch_kernel(attn_prefill_tcgen05_2q_kernel<64>, grid, dim3(kPPThreads), PPSmem<64>::kBytes, stream, map, p, skip_single);
    }
    return launch_status();
}
