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

}  // namespace cvb

using namespace cvb;

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
