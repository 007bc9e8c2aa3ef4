// Matrix products for a handful of tokens (decode steps of up to 16 rows), bf16 weights and activations:
//   y[m, n] = sum_k x[m, k] * W[n, k]
// With so few rows the product is a stream of the weight matrix through the SMs; a library GEMM leaves most of the
// HBM bandwidth unused at these shapes and cannot take the neighbouring elementwise work along.
//
// The weights are the A operand of mma.sync.m16n8k16 (16 or 8 rows of W per tile), the activations the B operand
// (8 columns = rows of x, zero-padded).  The sum over k does not care in which order k is walked, so every lane feeds
// the tensor core straight from 16-byte loads: lane (r = lane / 4, q = lane % 4) reads W[r][32j + 8q .. +7] and
// W[r + 8][same] from global memory and x[r][same] from shared memory, and the two k16 steps of a 32-wide slab use
// elements (0..3) and (4..7) of those vectors on both operands alike.  No conversion, no shuffle, no staging of W.
// A block holds a few tiles; the warps of a tile split K and add their partial sums through shared memory.
//
// Fused around the product (formulas of the reference's kernels/fused_ops.cu):
//   NORM      the activations are produced in the block itself: v = rnd(resid + delta) (written out once, by block 0,
//             as the new residual stream), x = rnd( rnd(v * rsqrt(mean(v^2) + eps)) * w )       (:61-88, add_rms_norm)
//   SWIGLU    W holds gate rows [0, I) and up rows [I, 2I); a tile is 8 gate rows over the 8 matching up rows and
//             the block stores T( rnd(silu(T(g))) * T(u) )                                      (:210-220)
// The result is rounded to bf16 once, as a library product with bf16 output is.
#include "common.cuh"
#include "sm100.cuh"

namespace cvb {

constexpr int kXPad = 32;              // elements of padding per activation row: rows land in different banks
constexpr int kBatch = 8;              // columns of the B operand
constexpr int kMaxRows = 16;           // activation rows a launch takes: one or two groups of kBatch
constexpr int kJBatch = 8;             // 32-wide slabs fetched ahead per warp

__device__ __forceinline__ void unpack8(const uint4& t, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct GemvParams {
    __nv_bfloat16* out;            // [M, N] (SWIGLU: [M, N / 2])
    const __nv_bfloat16* x;        // [M, K] activations (NORM: the residual stream)
    const __nv_bfloat16* delta;    // NORM: added to the residual first, or nullptr
    __nv_bfloat16* resid_out;      // NORM with delta: receives rnd(x + delta)
    const float* norm_w;           // NORM: [K]
    const __nv_bfloat16* W;        // [N, K]
    int M, N, K;
    int warps_k;                   // warps that share one tile's K range
    int tiles_per_block;           // tiles side by side in a block
    int n_tiles;
    float eps;
};

// TILE_ROWS: rows of W per tile (16, or 8 with the lower half of the A operand left zero).
// NB: activation rows in groups of eight (1 or 2): the B operand of a product holds eight rows, so sixteen rows take two
// products per weight fragment; the weights are still read once.
template <int TILE_ROWS, bool NORM, bool SWIGLU, int NB>
__global__ void __launch_bounds__(512)
gemv_mma_kernel(const GemvParams p) {
    constexpr int kRows = kBatch * NB;                                   // activation rows staged and multiplied
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K, chunks = K >> 3;
    const int xstride = K + kXPad;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [8][K + pad]
    float* red = reinterpret_cast<float*>(xs + kRows * xstride);                       // [warps][16][kRows]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    pdl_trigger();

    // ---- this warp's tiles and K range.  A block walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ... (each
    // `tiles_per_block` wide), so that the activations are staged once per block however many rows W has.  The first
    // batch of weights is fetched before anything else: weights do not depend on the kernels before this one, so the
    // fetch overlaps their tail and this kernel's own prologue ----
    constexpr int OUT_PER_TILE = SWIGLU ? 8 : TILE_ROWS;               // output columns a tile produces
    const int n_out = SWIGLU ? p.N / 2 : p.N;
    const int tile_in_block = warp / p.warps_k, wk = warp % p.warps_k;
    const int r = lane >> 2, q = lane & 3;
    constexpr bool LOWER = SWIGLU || TILE_ROWS == 16;
    const int slabs = (K + 31) >> 5;
    const int per_warp = (slabs + p.warps_k - 1) / p.warps_k;
    const int j_begin = wk * per_warp, j_end = min(slabs, j_begin + per_warp);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int n_rounds = (p.n_tiles + gridDim.x * p.tiles_per_block - 1) / (gridDim.x * p.tiles_per_block);
    int n0 = 0;
    const uint4 *w_hi = nullptr, *w_lo = nullptr;
    auto set_tile = [&](int round) {
        const int tile = (round * gridDim.x + blockIdx.x) * p.tiles_per_block + tile_in_block;
        n0 = tile * OUT_PER_TILE;
        // rows of W behind the upper (a0, a2) and lower (a1, a3) halves of the A operand
        int row_hi = n0 + r, row_lo = SWIGLU ? n_out + n0 + r : n0 + r + 8;
        row_hi = min(row_hi, p.N - 1);                                   // a ragged last tile repeats a row; dropped below
        row_lo = min(row_lo, p.N - 1);
        w_hi = reinterpret_cast<const uint4*>(p.W + static_cast<int64_t>(row_hi) * K);
        w_lo = reinterpret_cast<const uint4*>(p.W + static_cast<int64_t>(row_lo) * K);
    };
    uint4 wh[kJBatch], wl[kJBatch];
    auto fetch = [&](int jb) {
#pragma unroll
        for (int u = 0; u < kJBatch; ++u) {
            const int c = (jb + u) * 4 + q;                              // 16-byte chunk index along K
            const bool ok = n0 < n_out && jb + u < j_end && c < chunks;
            wh[u] = ok ? __ldg(w_hi + c) : zero;
            if constexpr (LOWER) wl[u] = ok ? __ldg(w_lo + c) : zero; else wl[u] = zero;
        }
    };
    set_tile(0);
    fetch(j_begin);
    pdl_wait();

    // ---- activations into shared memory ----
    // Loads come in batches of kStage per thread, all issued before the first of them is used: the staging then costs
    // about one trip to the L2 instead of one per loop iteration.
    constexpr int kStage = NORM ? 4 : 8;
    if constexpr (NORM) {
        // one warp per row: add, round, sum of squares, scale; the row passes through shared memory in between
        for (int m = warp; m < kRows; m += n_warps) {
            if (m >= p.M) {
                for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const uint4* xg = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(m) * K);
            const uint4* dg = p.delta != nullptr ? reinterpret_cast<const uint4*>(p.delta + static_cast<int64_t>(m) * K) : nullptr;
            float ss = 0.f;
            for (int c0 = lane; c0 < chunks; c0 += 32 * kStage) {
                uint4 xv[kStage], dv[kStage];
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = c0 + u * 32;
                    xv[u] = c < chunks ? xg[c] : zero;
                    dv[u] = (dg != nullptr && c < chunks) ? dg[c] : zero;
                }
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = c0 + u * 32;
                    if (c >= chunks) break;
                    float v[8];
                    unpack8(xv[u], v);
                    if (dg != nullptr) {
                        float d[8];
                        unpack8(dv[u], d);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = rnd<__nv_bfloat16>(v[i] + d[i]);
                    }
                    uint4 packed;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                    *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = packed;
                    if (dg != nullptr && blockIdx.x == 0)
                        *reinterpret_cast<uint4*>(p.resid_out + static_cast<int64_t>(m) * K + c * 8) = packed;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
                }
            }
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / static_cast<float>(K) + p.eps);
            for (int c0 = lane; c0 < chunks; c0 += 32 * kStage) {  // each lane re-reads the chunks it wrote itself
                float4 w0[kStage], w1[kStage];
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = min(c0 + u * 32, chunks - 1);
                    w0[u] = *reinterpret_cast<const float4*>(p.norm_w + c * 8);
                    w1[u] = *reinterpret_cast<const float4*>(p.norm_w + c * 8 + 4);
                }
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = c0 + u * 32;
                    if (c >= chunks) break;
                    float v[8];
                    unpack8(*reinterpret_cast<const uint4*>(xs + m * xstride + c * 8), v);
                    const float w[8] = {w0[u].x, w0[u].y, w0[u].z, w0[u].w, w1[u].x, w1[u].y, w1[u].z, w1[u].w};
                    uint4 packed;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        h[i] = __floats2bfloat162_rn(rnd<__nv_bfloat16>(v[2 * i] * inv) * w[2 * i],
                                                     rnd<__nv_bfloat16>(v[2 * i + 1] * inv) * w[2 * i + 1]);
                    *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = packed;
                }
            }
        }
    } else {
        const int total = kRows * chunks;
        for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * kStage) {
            uint4 v[kStage];
#pragma unroll
            for (int u = 0; u < kStage; ++u) {
                const int i = i0 + u * blockDim.x;
                const int m = i / chunks, c = i - m * chunks;
                v[u] = (i < total && m < p.M) ? *reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(m) * K + c * 8) : zero;
            }
#pragma unroll
            for (int u = 0; u < kStage; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i >= total) break;
                const int m = i / chunks, c = i - m * chunks;
                *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = v[u];
            }
        }
    }
    __syncthreads();

    // ---- the product, tile after tile ----
    const uint4* x_row[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) x_row[b] = reinterpret_cast<const uint4*>(xs + (r + 8 * b) * xstride);
    for (int round = 0; round < n_rounds; ++round) {
        float acc[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f; }
        for (int jb = j_begin; jb < j_end; jb += kJBatch) {
            if (jb != j_begin) fetch(jb);
#pragma unroll
            for (int u = 0; u < kJBatch; ++u) {
                const int c = (jb + u) * 4 + q;
                if (jb + u >= j_end) break;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const uint4 xv = c < chunks ? x_row[b][c] : zero;
                    mma_16816(acc[b], wh[u].x, wl[u].x, wh[u].y, wl[u].y, xv.x, xv.y);
                    mma_16816(acc[b], wh[u].z, wl[u].z, wh[u].w, wl[u].w, xv.z, xv.w);
                }
            }
        }
        const int tile_base = (round * gridDim.x + blockIdx.x) * p.tiles_per_block;
        if (round + 1 < n_rounds) {                                      // the next tile's weights are on their way
            set_tile(round + 1);                                         // while this one's parts are added up
            fetch(j_begin);
        }
        // acc[b][0], [1]: (row r, batch 8b + 2q, + 1); acc[b][2], [3]: (row r + 8, same)
        float* mine = red + warp * (16 * kRows);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            mine[r * kRows + 8 * b + 2 * q] = acc[b][0];
            mine[r * kRows + 8 * b + 2 * q + 1] = acc[b][1];
            mine[(r + 8) * kRows + 8 * b + 2 * q] = acc[b][2];
            mine[(r + 8) * kRows + 8 * b + 2 * q + 1] = acc[b][3];
        }
        __syncthreads();

        // ---- add the K parts of every tile and store ----
        for (int i = threadIdx.x; i < p.tiles_per_block * OUT_PER_TILE * kRows; i += blockDim.x) {
            const int t = i / (OUT_PER_TILE * kRows), rem = i % (OUT_PER_TILE * kRows);
            const int row = rem / kRows, m = rem % kRows;
            const int n = (tile_base + t) * OUT_PER_TILE + row;
            if (n >= n_out || m >= p.M) continue;
            float s0 = 0.f, s1 = 0.f;
            for (int w = 0; w < p.warps_k; ++w) {
                const float* part = red + (t * p.warps_k + w) * (16 * kRows);
                s0 += part[row * kRows + m];
                if constexpr (SWIGLU) s1 += part[(row + 8) * kRows + m];
            }
            float y = s0;
            if constexpr (SWIGLU) {
                const float g = rnd<__nv_bfloat16>(s0), u = rnd<__nv_bfloat16>(s1);
                y = rnd<__nv_bfloat16>(g / (1.f + expf(-g))) * u;
            }
            p.out[static_cast<int64_t>(m) * n_out + n] = __float2bfloat16_rn(y);
        }
        if (round + 1 < n_rounds) __syncthreads();                       // `red` is free again
    }
}

template <int TILE_ROWS, bool NORM, bool SWIGLU, int NB>
static int launch_gemv_nb(GemvParams p, cudaStream_t stream) {
    constexpr int OUT_PER_TILE = SWIGLU ? 8 : TILE_ROWS;
    const int n_out = SWIGLU ? p.N / 2 : p.N;
    const int tiles = (n_out + OUT_PER_TILE - 1) / OUT_PER_TILE;
    const int slabs = (p.K + 31) / 32;
    p.warps_k = max(1, min(16, (slabs + kJBatch - 1) / kJBatch));         // about one batch of loads per warp
    p.tiles_per_block = max(1, 8 / p.warps_k);
    while (p.tiles_per_block > 1 && (tiles + p.tiles_per_block - 1) / p.tiles_per_block < 120) p.tiles_per_block >>= 1;
    p.n_tiles = tiles;
    auto smem_for = [&](int tpb) {
        return static_cast<size_t>(kBatch * NB) * (p.K + kXPad) * sizeof(__nv_bfloat16) + static_cast<size_t>(p.warps_k * tpb) * 128 * NB * sizeof(float);
    };
    // Blocks stage all of the activations: with long rows few of them fit on an SM, and each then takes more warps
    // (up to 16) to keep as many loads in flight.  The grid is what the device holds at once; blocks walk the tiles.
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    if (smem_for(p.tiles_per_block) > 200 * 1024) return CVB_E_SIZE;
    auto resident = [&](int tpb) {                                   // blocks of this shape that an SM holds
        const size_t smem = smem_for(tpb);
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(gemv_mma_kernel<TILE_ROWS, NORM, SWIGLU, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess)
            return 0;
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_mma_kernel<TILE_ROWS, NORM, SWIGLU, NB>, p.warps_k * tpb * 32, smem) != cudaSuccess)
            return 0;
        return n;
    };
    int per_sm = resident(p.tiles_per_block);
    while (per_sm * p.warps_k * p.tiles_per_block < 16 && p.warps_k * p.tiles_per_block * 2 <= 16 &&
           smem_for(p.tiles_per_block * 2) <= 200 * 1024 && (tiles + p.tiles_per_block * 2 - 1) / (p.tiles_per_block * 2) >= sms) {
        p.tiles_per_block *= 2;
        per_sm = resident(p.tiles_per_block);
    }
    if (per_sm < 1) return CVB_E_SIZE;
    const int warps = p.warps_k * p.tiles_per_block;
    const int blocks = min((tiles + p.tiles_per_block - 1) / p.tiles_per_block, sms * per_sm);
    const size_t smem = smem_for(p.tiles_per_block);
    launch_kernel(gemv_mma_kernel<TILE_ROWS, NORM, SWIGLU, NB>, dim3(blocks), dim3(warps * 32), smem, stream, p);
    return launch_status();
}

// up to 8 rows: one group of eight; up to 16: two
template <int TILE_ROWS, bool NORM, bool SWIGLU>
static int launch_gemv(const GemvParams& p, cudaStream_t stream) {
    if (p.M <= kBatch) return launch_gemv_nb<TILE_ROWS, NORM, SWIGLU, 1>(p, stream);
    return launch_gemv_nb<TILE_ROWS, NORM, SWIGLU, 2>(p, stream);
}

template <bool NORM>
static int dispatch_gemv(const GemvParams& p, cudaStream_t stream) {
    // tiles of 16 rows while they still give about one block per SM, else tiles of 8
    if (p.N / 16 >= 120) return launch_gemv<16, NORM, false>(p, stream);
    return launch_gemv<8, NORM, false>(p, stream);
}

// ---- large weights: the inner dimension is split over blocks as well -----------------------------------------------
// The kernel above stages all of the activations in every block, which is right while W has a few thousand columns and a
// few MB.  For larger W a block takes kSkTiles tiles of 16 rows (one per warp) times one chunk of kSkChunk columns: 128 KB
// of weights behind 8 KB of staged activations, two batches of loads per warp, and enough blocks for every size.  The
// partial sums of the chunks go to a float scratch [chunk][batch row][N]; the block that finishes last among the chunks of
// its rows adds them up in chunk order (so the result does not depend on which block that was) and writes the output.
// `counters` holds one int per group of kSkTiles * 16 rows, zero before the first launch and zero again after each.
constexpr int kSkTiles = 8;
constexpr int kSkChunk = 512;
constexpr int kSkThreads = kSkTiles * 32;

struct SplitKParams {
    __nv_bfloat16* out;            // [M, N]
    const __nv_bfloat16* x;        // [M, K]
    const __nv_bfloat16* W;        // [N, K]
    float* part;                   // [splits, 8, N]
    int* counters;                 // [ceil(N / 128)]
    int M, N, K, splits;
};

__global__ void __launch_bounds__(kSkThreads, 2)
gemv_splitk_kernel(const SplitKParams p) {
    __shared__ __align__(16) __nv_bfloat16 xs[kBatch * (kSkChunk + kXPad)];
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
    const int K = p.K, chunks = K >> 3;
    const int k0 = blockIdx.y * kSkChunk;                                // first column of this block's chunk
    const int c0 = k0 >> 3, c_end = min(chunks, c0 + (kSkChunk >> 3));   // 16-byte chunks [c0, c_end)
    const int n0 = (blockIdx.x * kSkTiles + warp) * 16;
    pdl_trigger();
    const uint4* w_hi = reinterpret_cast<const uint4*>(p.W + static_cast<int64_t>(min(n0 + r, p.N - 1)) * K);
    const uint4* w_lo = reinterpret_cast<const uint4*>(p.W + static_cast<int64_t>(min(n0 + r + 8, p.N - 1)) * K);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 wh[kJBatch], wl[kJBatch];
    auto fetch = [&](int jb) {                                           // slabs jb .. jb + kJBatch - 1 of this chunk
#pragma unroll
        for (int u = 0; u < kJBatch; ++u) {
            const int c = c0 + (jb + u) * 4 + q;
            const bool ok = n0 < p.N && c < c_end;
            wh[u] = ok ? __ldg(w_hi + c) : zero;
            wl[u] = ok ? __ldg(w_lo + c) : zero;
        }
    };
    fetch(0);
    pdl_wait();
    constexpr int xstride = kSkChunk + kXPad;
    for (int i = threadIdx.x; i < kBatch * (kSkChunk >> 3); i += kSkThreads) {
        const int m = i / (kSkChunk >> 3), c = i % (kSkChunk >> 3);
        *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) =
            (m < p.M && c0 + c < c_end) ? *reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(m) * K + (c0 + c) * 8) : zero;
    }
    __syncthreads();
    const uint4* x_row = reinterpret_cast<const uint4*>(xs + r * xstride);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    constexpr int kSlabs = kSkChunk / 32;
#pragma unroll
    for (int jb = 0; jb < kSlabs; jb += kJBatch) {
        if (jb != 0) fetch(jb);
#pragma unroll
        for (int u = 0; u < kJBatch; ++u) {
            const uint4 xv = x_row[(jb + u) * 4 + q];
            mma_16816(acc, wh[u].x, wl[u].x, wh[u].y, wl[u].y, xv.x, xv.y);
            mma_16816(acc, wh[u].z, wl[u].z, wh[u].w, wl[u].w, xv.z, xv.w);
        }
    }
    // acc[0], acc[1]: (row r, batch 2q, 2q+1); acc[2], acc[3]: (row r + 8, same)
    float* part = p.part + static_cast<int64_t>(blockIdx.y) * kBatch * p.N;
    if (n0 + r < p.N) {
        part[static_cast<int64_t>(2 * q) * p.N + n0 + r] = acc[0];
        part[static_cast<int64_t>(2 * q + 1) * p.N + n0 + r] = acc[1];
    }
    if (n0 + r + 8 < p.N) {
        part[static_cast<int64_t>(2 * q) * p.N + n0 + r + 8] = acc[2];
        part[static_cast<int64_t>(2 * q + 1) * p.N + n0 + r + 8] = acc[3];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(p.counters + blockIdx.x, 1) == p.splits - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const int row0 = blockIdx.x * kSkTiles * 16;
    for (int i = threadIdx.x; i < p.M * kSkTiles * 16; i += kSkThreads) {
        const int m = i / (kSkTiles * 16), n = row0 + i % (kSkTiles * 16);
        if (n >= p.N) continue;
        const float* src = p.part + static_cast<int64_t>(m) * p.N + n;
        float sum = 0.f;
        int s = 0;
        for (; s + 4 <= p.splits; s += 4) {                              // four loads in flight, added in chunk order
            const float a = __ldcg(src + static_cast<int64_t>(s) * kBatch * p.N);
            const float b = __ldcg(src + static_cast<int64_t>(s + 1) * kBatch * p.N);
            const float c = __ldcg(src + static_cast<int64_t>(s + 2) * kBatch * p.N);
            const float d = __ldcg(src + static_cast<int64_t>(s + 3) * kBatch * p.N);
            sum = (((sum + a) + b) + c) + d;
        }
        for (; s < p.splits; ++s) sum += __ldcg(src + static_cast<int64_t>(s) * kBatch * p.N);
        p.out[static_cast<int64_t>(m) * p.N + n] = __float2bfloat16_rn(sum);
    }
    if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;
}


// ---- small models: one block per SM, the block's weights by bulk copy ahead of the dependency ------------------------
// When a weight matrix is a few megabytes, every block's share (N / #SMs rows of K elements) fits into its shared memory
// at once.  The kernel then asks for all of it with one bulk copy per row BEFORE it waits for the kernel in front of it
// (programmatic dependent launch: weights depend on no kernel), so that the weights travel while the predecessor still
// runs, and it lets its own successor start as soon as it has passed that wait.  What is left on the chain of dependent
// kernels is the trip of the activations through the L2 and the products themselves.  Blocks ask for about half of an
// SM's shared memory, so the blocks of two neighbouring kernels fit an SM together, one each.
// Rows land in shared memory with 64 bytes of padding, which makes the lanes' 16-byte reads (same k permutation as
// above) free of bank conflicts.  Arithmetic and rounding are those of the kernel above.
constexpr int kStWarps = 16;
constexpr int kStThreads = kStWarps * 32;

struct StreamParams {
    __nv_bfloat16* out;            // [M, N] (SWIGLU: [M, N / 2])
    const __nv_bfloat16* x;        // [M, K]
    const __nv_bfloat16* delta;    // NORM: added to the residual first, or nullptr
    __nv_bfloat16* resid_out;      // NORM with delta: receives rnd(x + delta)
    const float* norm_w;           // NORM: [K]
    const __nv_bfloat16* W;        // [N, K]
    const __nv_bfloat16* add_to;   // plain form: out = rnd(add_to + rnd(x W^T)) (the residual stream; may be `out` itself), or nullptr
    const unsigned char* prefetch; // bytes that a later kernel will stream: asked into the L2 by this one (or nullptr)
    long long prefetch_bytes;
    int* err;
    int M, N, K;
    int opb;                       // outputs per block
    int n_tiles;                   // tiles of 16 weight rows per block
    int warps_k;                   // warps that share one tile's K range
    int warps_per_row;             // NORM: warps that share one activation row (16 / rows, a power of two)
    int late_trigger;              // 1: the successor may start only when this block's products are done
    float eps;
};

// A load that the compiler may not move: issued where it stands (ahead of the dependency), used much later.
__device__ __forceinline__ float4 ld_early(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void bulk_row_to_smem(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem), "r"(bytes),
                   "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar))) : "memory");
}

// What runs after the wait is the chain that every decode step passes through once per product, so it is kept short:
// everything that can be worked out before the wait (addresses, which rows and outputs a thread owns, quotients) is,
// and no thread divides by a run-time number behind it.
// NB: groups of eight activation rows (1 or 2).  With two groups a block's shared memory may pass half an SM's, so
// one block runs per SM and a thread may hold twice the accumulators.
template <bool NORM, bool SWIGLU, int NB>
__global__ void __launch_bounds__(kStThreads, NB == 1 ? 2 : 1)
gemv_stream_kernel(const StreamParams p) {
    constexpr int kRowsX = kBatch * NB;                                            // activation rows staged
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = p.K, chunks = K >> 3, stride = K + kXPad;
    const int n_out = SWIGLU ? p.N / 2 : p.N;
    const int o0 = blockIdx.x * p.opb, n_mine = min(p.opb, n_out - o0);           // this block's outputs
    const int w_rows = SWIGLU ? 2 * n_mine : n_mine;
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
    float* row_ss = reinterpret_cast<float*>(smem_raw + 16);                       // [rows][16 parts]
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw + 16 + kRowsX * kStWarps * sizeof(float));   // [rows][K + pad]
    __nv_bfloat16* ws = xs + kRowsX * stride;                                      // [rows of W][K + pad]
    float* red = reinterpret_cast<float*>(ws + static_cast<size_t>(SWIGLU ? 2 : 1) * p.opb * stride);   // [item][16][rows]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4 zero = make_uint4(0, 0, 0, 0);

    // ---- before the dependency: the weights ----
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_expect_tx(bar, static_cast<uint32_t>(w_rows) * K * 2u);
    // One copy per row.  A warp issues the copies of its lanes one after the other, so the rows go round the warps.  (The
    // barrier's byte count may run ahead of the expectation above: its phase cannot end before thread 0 has arrived.)
    for (int r = warp + lane * kStWarps; r < w_rows; r += 32 * kStWarps) {
        const int grow = SWIGLU ? (r < n_mine ? o0 + r : n_out + o0 + (r - n_mine)) : o0 + r;
        bulk_row_to_smem(ws + static_cast<size_t>(r) * stride, p.W + static_cast<int64_t>(grow) * K, K * 2u, bar);
    }
    // ---- before the dependency: who does what afterwards ----
    // Activation row m belongs to the warps m * wpr .. m * wpr + wpr - 1 (wpr = 16 / rows, a power of two), each with a
    // range of the row's 16-byte chunks; a lane takes the chunks c_begin + lane, + 32, ...
    constexpr int kStage = 2;
    const int wpr = p.warps_per_row;
    const int my_row = warp / wpr, my_part = warp - my_row * wpr;
    const int per_part = (chunks + wpr - 1) / wpr;
    const int c_begin = my_part * per_part, c_end = min(chunks, c_begin + per_part);
    const bool has_row = my_row < p.M;
    const uint4* xg = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(has_row ? my_row : 0) * K);
    const uint4* dg = (NORM && p.delta != nullptr) ? reinterpret_cast<const uint4*>(p.delta + static_cast<int64_t>(has_row ? my_row : 0) * K) : nullptr;
    uint4* xs_row = reinterpret_cast<uint4*>(xs + my_row * stride);
    float4 nw0[kStage], nw1[kStage];
    if constexpr (NORM) {
#pragma unroll
        for (int u = 0; u < kStage; ++u) {
            const int c = min(c_begin + lane + u * 32, chunks - 1);
            nw0[u] = ld_early(p.norm_w + c * 8);
            nw1[u] = ld_early(p.norm_w + c * 8 + 4);
        }
    }
    // the products: a warp's first (tile, K range) item and the rows of W behind the two halves of the A operand
    constexpr int OUT_PER_TILE = SWIGLU ? 8 : 16;
    const int r = lane >> 2, q = lane & 3;
    const int slabs = (K + 31) >> 5;
    const int per_warp = (slabs + p.warps_k - 1) / p.warps_k;
    const int items = p.n_tiles * p.warps_k;
    // B operand: column r of a product is activation row r; columns without a token repeat the last row and are not stored
    const uint4* x_row = reinterpret_cast<const uint4*>(xs + min(r, p.M - 1) * stride);
    const uint4* x_row_b = reinterpret_cast<const uint4*>(xs + min(r + kBatch, p.M - 1) * stride);   // second group (NB == 2)
    auto rows_of = [&](int tile, const uint4*& w_hi, const uint4*& w_lo) {
        int row_hi, row_lo;
        if constexpr (SWIGLU) {
            row_hi = min(tile * 8 + r, n_mine - 1);
            row_lo = n_mine + row_hi;
        } else {
            row_hi = min(tile * 16 + r, n_mine - 1);
            row_lo = min(tile * 16 + r + 8, n_mine - 1);
        }
        w_hi = reinterpret_cast<const uint4*>(ws + static_cast<size_t>(row_hi) * stride);
        w_lo = reinterpret_cast<const uint4*>(ws + static_cast<size_t>(row_lo) * stride);
    };
    int tile = warp / p.warps_k, wk = warp - tile * p.warps_k;
    const uint4 *w_hi, *w_lo;
    rows_of(tile, w_hi, w_lo);
    // the store: thread i takes output i % n_mine of row i / n_mine
    int e_m = threadIdx.x / n_mine, e_o = threadIdx.x - e_m * n_mine;
    const float inv_k = 1.f / static_cast<float>(K);
    pdl_wait();
    // the residual element that this thread's first output is added to: asked for now, used at the very end
    float res_first = 0.f;
    if (p.add_to != nullptr && threadIdx.x < p.M * n_mine)
        res_first = __bfloat162float(__ldcg(p.add_to + static_cast<int64_t>(e_m) * n_out + o0 + e_o));

    // ---- activations into shared memory (read past the L1: another kernel wrote them while this block was resident) ----
    if constexpr (NORM) {
        float ss = 0.f;
        uint4 keep[kStage];                                              // the first pass's chunks stay in registers
        if (has_row) {
            for (int c0 = c_begin + lane; c0 < c_end; c0 += 32 * kStage) {
                uint4 xv[kStage], dv[kStage];
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = c0 + u * 32;
                    xv[u] = c < c_end ? __ldcg(xg + c) : zero;
                    dv[u] = (dg != nullptr && c < c_end) ? __ldcg(dg + c) : zero;
                }
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = c0 + u * 32;
                    // rnd(x + delta) two at a time: the packed addition rounds the exact sum once, as the float one does
                    uint4 packed = xv[u];
                    if (dg != nullptr) {
                        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&packed);
                        const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[u]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) a2[i] = __hadd2(a2[i], d2[i]);
                    }
                    if (c0 == c_begin + lane) keep[u] = packed;
                    else if (c < c_end) xs_row[c] = packed;              // later passes wait in shared memory
                    if (dg != nullptr && blockIdx.x == 0 && c < c_end)
                        *reinterpret_cast<uint4*>(p.resid_out + static_cast<int64_t>(my_row) * K + c * 8) = packed;
                    float v[8];
                    unpack8(packed, v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);   // chunks past the end are zero
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) row_ss[my_row * kStWarps + my_part] = ss;
        }
        __syncthreads();
        if (has_row) {
            // the row's parts, one per lane, added by the same tree in every warp and block
            float total = warp_sum(lane < wpr ? row_ss[my_row * kStWarps + lane] : 0.f);
            const float inv = rsqrtf(total * inv_k + p.eps);
            for (int c0 = c_begin + lane; c0 < c_end; c0 += 32 * kStage) {
                const bool first = c0 == c_begin + lane;
                if (!first) {
#pragma unroll
                    for (int u = 0; u < kStage; ++u) {
                        const int c = min(c0 + u * 32, chunks - 1);
                        nw0[u] = __ldg(reinterpret_cast<const float4*>(p.norm_w + c * 8));
                        nw1[u] = __ldg(reinterpret_cast<const float4*>(p.norm_w + c * 8 + 4));
                    }
                }
#pragma unroll
                for (int u = 0; u < kStage; ++u) {
                    const int c = c0 + u * 32;
                    if (c >= c_end) break;
                    float v[8];
                    unpack8(first ? keep[u] : xs_row[c], v);
                    const float w[8] = {nw0[u].x, nw0[u].y, nw0[u].z, nw0[u].w, nw1[u].x, nw1[u].y, nw1[u].z, nw1[u].w};
                    uint4 packed;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        h[i] = __floats2bfloat162_rn(rnd<__nv_bfloat16>(v[2 * i] * inv) * w[2 * i],
                                                     rnd<__nv_bfloat16>(v[2 * i + 1] * inv) * w[2 * i + 1]);
                    xs_row[c] = packed;
                }
            }
        }
    } else {
        if (has_row) {
            constexpr int kCopy = 4;
            for (int c0 = c_begin + lane; c0 < c_end; c0 += 32 * kCopy) {
                uint4 v[kCopy];
#pragma unroll
                for (int u = 0; u < kCopy; ++u) v[u] = c0 + u * 32 < c_end ? __ldcg(xg + c0 + u * 32) : zero;
#pragma unroll
                for (int u = 0; u < kCopy; ++u)
                    if (c0 + u * 32 < c_end) xs_row[c0 + u * 32] = v[u];
            }
        }
    }
    __syncthreads();
    // The successor's blocks arrive on this SM and ask for their weights at once: only now, when this block's own
    // activations have come in, so that they do not queue behind those weights.
    if (!p.late_trigger) pdl_trigger();
    if (p.prefetch != nullptr && threadIdx.x == 32) {
        // this block's share of what a later kernel streams, in pieces of at most 64 KB
        const long long share = ((p.prefetch_bytes + gridDim.x - 1) / gridDim.x + 15) & ~15LL;
        const long long begin = share * blockIdx.x, end = min(p.prefetch_bytes & ~15LL, begin + share);
        for (long long o = begin; o < end; o += 65536) {
            const uint32_t n = static_cast<uint32_t>(min(65536LL, end - o));
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p.prefetch + o), "r"(n) : "memory");
        }
    }
    mbar_wait(bar, 0, p.err);

    // ---- the products: a warp takes (tile, K range) items; four independent chains of products ----
    for (int item = warp; item < items; item += kStWarps) {
        if (item != warp) {
            tile = item / p.warps_k;
            wk = item - tile * p.warps_k;
            rows_of(tile, w_hi, w_lo);
        }
        float acc[4][4], acc_b[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            acc_b[i][0] = acc_b[i][1] = acc_b[i][2] = acc_b[i][3] = 0.f;
        }
        const int j_end = min(slabs, (wk + 1) * per_warp);
        int c = wk * per_warp * 4 + q;
        for (int j0 = wk * per_warp; j0 < j_end; j0 += 2, c += 8) {
            const bool ok0 = c < chunks, ok1 = j0 + 1 < j_end && c + 4 < chunks;
            const uint4 wh0 = ok0 ? w_hi[c] : zero, wl0 = ok0 ? w_lo[c] : zero, xv0 = ok0 ? x_row[c] : zero;
            const uint4 wh1 = ok1 ? w_hi[c + 4] : zero, wl1 = ok1 ? w_lo[c + 4] : zero, xv1 = ok1 ? x_row[c + 4] : zero;
            mma_16816(acc[0], wh0.x, wl0.x, wh0.y, wl0.y, xv0.x, xv0.y);
            mma_16816(acc[1], wh0.z, wl0.z, wh0.w, wl0.w, xv0.z, xv0.w);
            mma_16816(acc[2], wh1.x, wl1.x, wh1.y, wl1.y, xv1.x, xv1.y);
            mma_16816(acc[3], wh1.z, wl1.z, wh1.w, wl1.w, xv1.z, xv1.w);
            if constexpr (NB == 2) {                                 // the same weight fragments against rows 8 .. 15
                const uint4 xb0 = ok0 ? x_row_b[c] : zero, xb1 = ok1 ? x_row_b[c + 4] : zero;
                mma_16816(acc_b[0], wh0.x, wl0.x, wh0.y, wl0.y, xb0.x, xb0.y);
                mma_16816(acc_b[1], wh0.z, wl0.z, wh0.w, wl0.w, xb0.z, xb0.w);
                mma_16816(acc_b[2], wh1.x, wl1.x, wh1.y, wl1.y, xb1.x, xb1.y);
                mma_16816(acc_b[3], wh1.z, wl1.z, wh1.w, wl1.w, xb1.z, xb1.w);
            }
        }
        // acc[.][0], [1]: (row r, batch 2q, 2q + 1); acc[.][2], [3]: (row r + 8, same)
        float* mine = red + item * (128 * NB);
        mine[r * kRowsX + 2 * q] = (acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0]);
        mine[r * kRowsX + 2 * q + 1] = (acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1]);
        mine[(r + 8) * kRowsX + 2 * q] = (acc[0][2] + acc[1][2]) + (acc[2][2] + acc[3][2]);
        mine[(r + 8) * kRowsX + 2 * q + 1] = (acc[0][3] + acc[1][3]) + (acc[2][3] + acc[3][3]);
        if constexpr (NB == 2) {
            mine[r * kRowsX + 8 + 2 * q] = (acc_b[0][0] + acc_b[1][0]) + (acc_b[2][0] + acc_b[3][0]);
            mine[r * kRowsX + 8 + 2 * q + 1] = (acc_b[0][1] + acc_b[1][1]) + (acc_b[2][1] + acc_b[3][1]);
            mine[(r + 8) * kRowsX + 8 + 2 * q] = (acc_b[0][2] + acc_b[1][2]) + (acc_b[2][2] + acc_b[3][2]);
            mine[(r + 8) * kRowsX + 8 + 2 * q + 1] = (acc_b[0][3] + acc_b[1][3]) + (acc_b[2][3] + acc_b[3][3]);
        }
    }
    __syncthreads();
    if (p.late_trigger) pdl_trigger();

    // ---- add the K parts and store: consecutive threads, consecutive outputs ----
    for (int i = threadIdx.x; i < p.M * n_mine; i += kStThreads) {
        if (i != static_cast<int>(threadIdx.x)) { e_m = i / n_mine; e_o = i - e_m * n_mine; }
        const int t = e_o / OUT_PER_TILE, row = e_o - t * OUT_PER_TILE;
        const float* part = red + t * p.warps_k * (128 * NB) + row * kRowsX + e_m;
        float s0 = 0.f, s1 = 0.f;
        for (int w = 0; w < p.warps_k; ++w) {
            s0 += part[w * (128 * NB)];
            if constexpr (SWIGLU) s1 += part[w * (128 * NB) + 64 * NB];
        }
        float y = s0;
        if constexpr (SWIGLU) {
            const float g = rnd<__nv_bfloat16>(s0), u = rnd<__nv_bfloat16>(s1);
            y = rnd<__nv_bfloat16>(g / (1.f + expf(-g))) * u;
        }
        if (p.add_to != nullptr) {                                   // the residual sum, rounded where the separate kernels round
            const float res = i == static_cast<int>(threadIdx.x) ? res_first
                                                                 : __bfloat162float(__ldcg(p.add_to + static_cast<int64_t>(e_m) * n_out + o0 + e_o));
            y = res + rnd<__nv_bfloat16>(y);
        }
        p.out[static_cast<int64_t>(e_m) * n_out + o0 + e_o] = __float2bfloat16_rn(y);
    }
}

// The plan of a launch: outputs per block, tiles, warps per tile and shared memory; false if the shape is not for this
// kernel (the block's rows do not fit into about half an SM's shared memory).
struct StreamPlan { int blocks, opb, n_tiles, warps_k; size_t smem; };
static bool stream_plan(int N, int K, bool swiglu, int nb, StreamPlan* plan) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int n_out = swiglu ? N / 2 : N;
    if (n_out <= 0 || K <= 0 || (K % 8) || (swiglu && (N % 2))) return false;
    const int opb = (n_out + sms - 1) / sms;
    const int per_tile = swiglu ? 8 : 16;
    const int n_tiles = (opb + per_tile - 1) / per_tile;
    const int slabs = (K + 31) / 32;
    const int warps_k = max(1, min(slabs, kStWarps / n_tiles));
    const size_t row = static_cast<size_t>(K + kXPad) * sizeof(__nv_bfloat16);
    const size_t smem = 16 + static_cast<size_t>(kBatch) * nb * kStWarps * sizeof(float) +
                        row * (static_cast<size_t>(kBatch) * nb + static_cast<size_t>(swiglu ? 2 : 1) * opb) +
                        static_cast<size_t>(n_tiles) * warps_k * 128 * nb * sizeof(float);
    // up to eight rows: half an SM's shared memory, so that a block of the next kernel fits beside this one; nine to
    // sixteen rows: whatever an SM has
    if (smem > (nb == 1 ? 113u : 226u) * 1024 || static_cast<size_t>(swiglu ? 2 : 1) * opb * K * 2 >= (1u << 20)) return false;
    plan->blocks = (n_out + opb - 1) / opb; plan->opb = opb; plan->n_tiles = n_tiles; plan->warps_k = warps_k; plan->smem = smem;
    return true;
}


// ---- large weights: one block per SM, the block's rows streamed through a ring of bulk copies ------------------------
// A weight of tens or hundreds of megabytes is a stream that must keep every SM's memory pipe full from the first
// microsecond to the last.  Block b owns the rows [b N / G, (b + 1) N / G) of W (whole rows, so no partial sums cross
// blocks, and the split is even to a row) and walks them in tiles of 16 rows times chunks of kRingK columns.  Four
// producer warps bring a tile's chunk (one bulk copy per row piece, 2 KB) and the same chunk of the activations (from
// the L2) into one of kRingStages stages; eight consumer warps each multiply an eighth of the chunk's columns (the same
// fragments as above) and keep their partial sums in registers across the chunks of a tile; at the tile's end the eight
// parts are added through shared memory.  The first stages' weights are asked for ahead of griddepcontrol.wait.
constexpr int kRingK = 1024;                 // columns per chunk
constexpr int kRingStages = 4;
constexpr int kRingConsumers = 8;            // warps
constexpr int kRingProducers = 4;            // warps (a warp issues its lanes' copies one after the other)
constexpr int kRingThreads = (kRingConsumers + kRingProducers) * 32;
constexpr int kRingRowBytes = kRingK * 2 + 64;                       // a row piece in shared memory, padded
constexpr int kRingStageBytes = (16 + kBatch) * kRingRowBytes;       // 16 rows of W, then 8 rows of x
constexpr size_t kRingSmem = 128 + static_cast<size_t>(kRingStages) * kRingStageBytes + kRingConsumers * 16 * kBatch * sizeof(float);

struct RingParams {
    __nv_bfloat16* out;            // [M, N]
    const __nv_bfloat16* x;        // [M, K]
    const __nv_bfloat16* W;        // [N, K]
    int* err;
    int M, N, K;
};

__global__ void __launch_bounds__(kRingThreads, 1)
gemv_ring_kernel(const RingParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);                 // [stages]: the copies of a stage have landed
    uint64_t* empty = full + kRingStages;                                    // [stages]: the eight consumer warps are done with it
    unsigned char* stages = smem_raw + 128;
    float* red = reinterpret_cast<float*>(stages + static_cast<size_t>(kRingStages) * kRingStageBytes);   // [8][16][8]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = p.K;
    const int row0 = static_cast<int>(static_cast<long long>(blockIdx.x) * p.N / gridDim.x);
    const int row1 = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * p.N / gridDim.x);
    const int n_tiles = (row1 - row0 + 15) >> 4;
    const int n_chunks = (K + kRingK - 1) / kRingK;
    const int total = n_tiles * n_chunks;                                    // stages' worth of work, tile-major
    if (threadIdx.x == 0) {
        for (int i = 0; i < kRingStages; ++i) { mbar_init(full + i, kRingProducers); mbar_init(empty + i, kRingConsumers); }
        mbar_fence_init();
    }
    __syncthreads();
    if (warp >= kRingConsumers) {
        // ---- producers: each of the four warps brings four rows of a tile (lanes 0..3) and two activation rows (lanes 4, 5) ----
        constexpr int kWRows = 16 / kRingProducers, kXRows = kBatch / kRingProducers;
        const int pw = warp - kRingConsumers;
        const int w_row = pw * kWRows + lane;
        const int x_row = pw * kXRows + (lane - kWRows);
        auto bytes_of = [&](int it) {                                        // what this warp brings for item `it`
            const int tile = it / n_chunks, chunk = it - tile * n_chunks;
            const uint32_t piece = static_cast<uint32_t>(min(kRingK, K - chunk * kRingK)) * 2u;
            const int rows_here = max(0, min(kWRows, row1 - row0 - tile * 16 - pw * kWRows));
            const int x_here = max(0, min(kXRows, p.M - pw * kXRows));
            return piece * static_cast<uint32_t>(rows_here + x_here);
        };
        auto issue = [&](int it, bool weights, bool acts) {
            const int tile = it / n_chunks, chunk = it - tile * n_chunks;
            const int st = it % kRingStages;
            const uint32_t piece = static_cast<uint32_t>(min(kRingK, K - chunk * kRingK)) * 2u;
            unsigned char* base = stages + static_cast<size_t>(st) * kRingStageBytes;
            if (weights && lane < kWRows) {
                const int row = row0 + tile * 16 + w_row;
                if (row < row1)
                    bulk_row_to_smem(base + w_row * kRingRowBytes, p.W + static_cast<int64_t>(row) * K + chunk * kRingK, piece, full + st);
            }
            if (acts && lane >= kWRows && lane < kWRows + kXRows && x_row < p.M)
                bulk_row_to_smem(base + (16 + x_row) * kRingRowBytes, p.x + static_cast<int64_t>(x_row) * K + chunk * kRingK, piece, full + st);
        };
        const int ahead = min(kRingStages, total);
        for (int it = 0; it < ahead; ++it) {                                 // weights depend on no kernel: before the wait
            if (lane == 0) mbar_expect_tx(full + it, bytes_of(it));
            __syncwarp();
            issue(it, true, false);
        }
        pdl_wait();
        for (int it = 0; it < ahead; ++it) issue(it, false, true);           // the activations: behind it
        for (int it = ahead; it < total; ++it) {
            const int st = it % kRingStages;
            if (lane == 0) {
                mbar_wait(empty + st, ((it / kRingStages) - 1) & 1, p.err);
                mbar_expect_tx(full + st, bytes_of(it));
            }
            __syncwarp();
            issue(it, true, true);
        }
        pdl_trigger();
        return;
    }
    // ---- consumers ----
    pdl_wait();
    const int r = lane >> 2, q = lane & 3;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    int it = 0;
    for (int tile = 0; tile < n_tiles; ++tile) {
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const int rows_here = min(16, row1 - row0 - tile * 16);
        for (int chunk = 0; chunk < n_chunks; ++chunk, ++it) {
            const int st = it % kRingStages;
            mbar_wait(full + st, (it / kRingStages) & 1, p.err);
            const unsigned char* base = stages + static_cast<size_t>(st) * kRingStageBytes;
            // rows past the block's last row were not copied: their lanes read the tile's last row, and are not stored
            const uint4* w_hi = reinterpret_cast<const uint4*>(base + min(r, rows_here - 1) * kRingRowBytes);
            const uint4* w_lo = reinterpret_cast<const uint4*>(base + min(r + 8, rows_here - 1) * kRingRowBytes);
            const uint4* xs = reinterpret_cast<const uint4*>(base + (16 + min(r, p.M - 1)) * kRingRowBytes);
            const int n16 = min(kRingK, K - chunk * kRingK) >> 3;            // 16-byte pieces in this chunk's rows
#pragma unroll
            for (int j = 0; j < kRingK / 32 / kRingConsumers; j += 2) {      // this warp's slabs of 32 columns, two at a time
                const int c0 = (warp * (kRingK / 32 / kRingConsumers) + j) * 4 + q, c1 = c0 + 4;
                const bool ok0 = c0 < n16, ok1 = c1 < n16;
                const uint4 wh0 = ok0 ? w_hi[c0] : zero, wl0 = ok0 ? w_lo[c0] : zero, xv0 = ok0 ? xs[c0] : zero;
                const uint4 wh1 = ok1 ? w_hi[c1] : zero, wl1 = ok1 ? w_lo[c1] : zero, xv1 = ok1 ? xs[c1] : zero;
                mma_16816(acc[0], wh0.x, wl0.x, wh0.y, wl0.y, xv0.x, xv0.y);
                mma_16816(acc[1], wh0.z, wl0.z, wh0.w, wl0.w, xv0.z, xv0.w);
                mma_16816(acc[0], wh1.x, wl1.x, wh1.y, wl1.y, xv1.x, xv1.y);
                mma_16816(acc[1], wh1.z, wl1.z, wh1.w, wl1.w, xv1.z, xv1.w);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);
        }
        // the tile is complete: add the eight warps' parts (acc[.][0], [1]: row r, batch 2q, 2q + 1; [2], [3]: row r + 8)
        float* mine = red + warp * 128;
        mine[r * 8 + 2 * q] = acc[0][0] + acc[1][0];
        mine[r * 8 + 2 * q + 1] = acc[0][1] + acc[1][1];
        mine[(r + 8) * 8 + 2 * q] = acc[0][2] + acc[1][2];
        mine[(r + 8) * 8 + 2 * q + 1] = acc[0][3] + acc[1][3];
        asm volatile("bar.sync 1, %0;\n" ::"n"(kRingConsumers * 32) : "memory");
        if (threadIdx.x < 128) {
            const int m = threadIdx.x >> 4, row = threadIdx.x & 15;          // consecutive threads, consecutive outputs
            if (m < p.M && row < rows_here) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kRingConsumers; ++w) sum += red[w * 128 + row * 8 + m];
                p.out[static_cast<int64_t>(m) * p.N + row0 + tile * 16 + row] = __float2bfloat16_rn(sum);
            }
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(kRingConsumers * 32) : "memory");      // `red` is free again
    }
}

}  // namespace cvb

using namespace cvb;

// 1 if cvb_gemv_stream_bf16 takes a weight of N rows and K columns in this mode (0 plain, 1 norm, 2 norm + SwiGLU)
// for `rows` activation rows.
extern "C" int cvb_gemv_stream_supported(int N, int K, int mode, int rows) {
    StreamPlan plan;
    return rows > 0 && rows <= 2 * kBatch && stream_plan(N, K, mode == 2, rows > kBatch ? 2 : 1, &plan) ? 1 : 0;
}

// out[:M] = x[:M] W^T for up to 16 rows and a weight whose per-SM share fits into shared memory; modes as cvb_gemv_bf16.
// `add_to` (plain mode; or null): out = rnd(add_to + rnd(x W^T)), the residual sum folded into the store (add_to may be out).
// `prefetch` (or null) names bytes that a later kernel will stream; this one asks them into the L2.  With `late_trigger`
// the kernel behind this one starts when this one's products are done rather than as early as possible.  The launch
// always carries the programmatic-dependent-launch attribute unless `pdl` is 0.
extern "C" int cvb_gemv_stream_bf16(void* out, const void* x, const void* delta, void* resid_out, const float* norm_w,
                                    const void* W, int M, int N, int K, float eps, int mode, const void* add_to, const void* prefetch,
                                    long long prefetch_bytes, int late_trigger, int pdl, int* err, cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || M > 2 * kBatch || N <= 0 || K <= 0) return CVB_E_SIZE;
    if (K % 8) return CVB_E_ALIGN;
    const int nb = M > kBatch ? 2 : 1;
    auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(out) || !al(x) || !al(delta) || !al(resid_out) || !al(W) || !al(norm_w) || !al(prefetch)) return CVB_E_ALIGN;
    if (mode != 0 && norm_w == nullptr) return CVB_E_SHAPE;
    if (mode < 0 || mode > 2 || err == nullptr) return CVB_E_SHAPE;
    if (delta != nullptr && (resid_out == nullptr || resid_out == x)) return CVB_E_SHAPE;
    if (add_to != nullptr && (mode != 0 || (reinterpret_cast<uintptr_t>(add_to) & 1))) return CVB_E_SHAPE;
    StreamPlan plan;
    if (!stream_plan(N, K, mode == 2, nb, &plan)) return CVB_E_UNSUPPORTED;
    StreamParams p{};
    p.out = (__nv_bfloat16*)out; p.x = (const __nv_bfloat16*)x; p.delta = (const __nv_bfloat16*)delta;
    p.resid_out = (__nv_bfloat16*)resid_out; p.norm_w = norm_w; p.W = (const __nv_bfloat16*)W;
    p.add_to = (const __nv_bfloat16*)add_to;
    p.prefetch = (const unsigned char*)prefetch; p.prefetch_bytes = prefetch != nullptr ? prefetch_bytes : 0; p.err = err;
    p.M = M; p.N = N; p.K = K; p.opb = plan.opb; p.n_tiles = plan.n_tiles; p.warps_k = plan.warps_k;
    p.late_trigger = late_trigger ? 1 : 0; p.eps = eps;
    // warps that share an activation row in the norm prologue: 16 / rows, but no more than give every lane a chunk (warps
    // without work go straight to the barrier and leave the issue slots to those that have some)
    p.warps_per_row = M <= 1 ? 16 : (M <= 2 ? 8 : (M <= 4 ? 4 : (M <= 8 ? 2 : 1)));
    while (p.warps_per_row > 1 && (K / 8 + 31) / 32 < p.warps_per_row) p.warps_per_row >>= 1;
    static bool set[6] = {false, false, false, false, false, false};   // the kernels share one pointer type: one flag per (mode, groups)
    auto go = [&](void (*kernel)(StreamParams)) {
        const int which = mode + 3 * (nb - 1);
        if (!set[which]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (nb == 1 ? 113 : 226) * 1024) != cudaSuccess) { cudaGetLastError(); return CVB_E_SIZE; }
            // all kernels of the chain ask for the largest shared-memory partition, so that a block of the next kernel
            // can join a running block on its SM without the partition having to change
            cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaGetLastError();
            set[which] = true;
        }
        launch_kernel_dependent(kernel, dim3(plan.blocks), dim3(kStThreads), plan.smem, stream, pdl != 0, p);
        return launch_status();
    };
    if (nb == 1) {
        if (mode == 0) return go(gemv_stream_kernel<false, false, 1>);
        if (mode == 1) return go(gemv_stream_kernel<true, false, 1>);
        return go(gemv_stream_kernel<true, true, 1>);
    }
    if (mode == 0) return go(gemv_stream_kernel<false, false, 2>);
    if (mode == 1) return go(gemv_stream_kernel<true, false, 2>);
    return go(gemv_stream_kernel<true, true, 2>);
}


// mode: 0 = plain product, 1 = norm(+add) prologue, 2 = norm(+add) prologue and SwiGLU epilogue.
extern "C" int cvb_gemv_bf16(void* out, const void* x, const void* delta, void* resid_out, const float* norm_w,
                             const void* W, int M, int N, int K, float eps, int mode, cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || M > kMaxRows || N <= 0 || K <= 0) return CVB_E_SIZE;
    if (K % 8) return CVB_E_ALIGN;
    auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(out) || !al(x) || !al(delta) || !al(resid_out) || !al(W) || !al(norm_w)) return CVB_E_ALIGN;
    if (mode != 0 && norm_w == nullptr) return CVB_E_SHAPE;
    if (delta != nullptr && (resid_out == nullptr || resid_out == x)) return CVB_E_SHAPE;   // blocks read x while block 0 writes
    if (mode == 2 && (N % 2)) return CVB_E_SHAPE;
    GemvParams p{};
    p.out = (__nv_bfloat16*)out; p.x = (const __nv_bfloat16*)x; p.delta = (const __nv_bfloat16*)delta;
    p.resid_out = (__nv_bfloat16*)resid_out; p.norm_w = norm_w; p.W = (const __nv_bfloat16*)W;
    p.M = M; p.N = N; p.K = K; p.eps = eps;
    if (mode == 0) return dispatch_gemv<false>(p, stream);
    if (mode == 1) return dispatch_gemv<true>(p, stream);
    if (mode == 2) return launch_gemv<16, true, true>(p, stream);
    return CVB_E_SHAPE;
}

// Floats of scratch and ints of counters that cvb_gemv_splitk_bf16 needs for a weight of N rows and K columns.
extern "C" int64_t cvb_gemv_splitk_scratch_floats(int N, int K) {
    return static_cast<int64_t>((K + kSkChunk - 1) / kSkChunk) * kBatch * N;
}
extern "C" int cvb_gemv_splitk_counters(int N) { return (N + kSkTiles * 16 - 1) / (kSkTiles * 16); }

// out[:M] = x[:M] W^T for up to 8 rows, the inner dimension split over blocks (for large W).
extern "C" int cvb_gemv_splitk_bf16(void* out, const void* x, const void* W, int M, int N, int K, float* scratch,
                                    int64_t scratch_floats, int* counters, cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || M > kBatch || N <= 0 || K <= 0) return CVB_E_SIZE;
    if (K % 8) return CVB_E_ALIGN;
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(out) || !al(x) || !al(W)) return CVB_E_ALIGN;
    if (scratch == nullptr || counters == nullptr || scratch_floats < cvb_gemv_splitk_scratch_floats(N, K)) return CVB_E_SCRATCH;
    SplitKParams p{};
    p.out = (__nv_bfloat16*)out; p.x = (const __nv_bfloat16*)x; p.W = (const __nv_bfloat16*)W;
    p.part = scratch; p.counters = counters; p.M = M; p.N = N; p.K = K;
    p.splits = (K + kSkChunk - 1) / kSkChunk;
    if (p.splits > 65535) return CVB_E_SIZE;
    dim3 grid(static_cast<unsigned>(cvb_gemv_splitk_counters(N)), static_cast<unsigned>(p.splits));
    launch_kernel(gemv_splitk_kernel, grid, dim3(kSkThreads), 0, stream, p);
    return launch_status();
}

// out[:M] = x[:M] W^T for up to 8 rows and a weight of any size, streamed through a ring of shared-memory stages by one
// block per SM (see gemv_ring_kernel).  `dependent`: launch with the programmatic-dependent-launch attribute.
extern "C" int cvb_gemv_ring_bf16(void* out, const void* x, const void* W, int M, int N, int K, int dependent, int* err,
                                  cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || M > kBatch || N <= 0 || K <= 0) return CVB_E_SIZE;
    if (K % 8) return CVB_E_ALIGN;
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(out) || !al(x) || !al(W)) return CVB_E_ALIGN;
    if (err == nullptr) return CVB_E_SHAPE;
    static int sms = 0;
    static bool set = false;
    if (!set) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaFuncSetAttribute(gemv_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRingSmem)) != cudaSuccess) {
            cudaGetLastError();
            return CVB_E_SIZE;
        }
        set = true;
    }
    RingParams p{};
    p.out = (__nv_bfloat16*)out; p.x = (const __nv_bfloat16*)x; p.W = (const __nv_bfloat16*)W; p.err = err;
    p.M = M; p.N = N; p.K = K;
    const int blocks = min(sms > 0 ? sms : 148, N);
    launch_kernel_dependent(gemv_ring_kernel, dim3(blocks), dim3(kRingThreads), kRingSmem, stream, dependent != 0, p);
    return launch_status();
}
