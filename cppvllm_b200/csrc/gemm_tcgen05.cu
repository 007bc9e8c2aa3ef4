// Matrix product on the fifth-generation tensor cores (tcgen05) for prompt portions, bf16:
//   C[M, N] = A[M, K] * W[N, K]^T          (A activations, W a weight matrix as checkpoints store it; both K-major)
// and its fused form for the gated feed-forward:
//   C[M, I] = T( rnd(silu(T(G))) * T(U) ),  G = A * W[0:I]^T,  U = A * W[I:2I]^T      (kernels/fused_ops.cu:210-220 of
//   the reference), where one tile's B operand is 128 gate rows over the 128 matching up rows, so that gate and up
//   of a column end up in the same accumulator row and the activations never travel through global memory.
//
// The kernel is persistent: one block per SM walks the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... in an order
// (tile_origin) in which the blocks that run side by side share the activations and the weight rows they read.
// Roles, by warp:
//   warp 0   producer: one thread issues TMA copies (cp.async.bulk.tensor.2d, 128-byte swizzle) of the A tile [128 x 64]
//            and the B tile [BN x 64] of every k-block of every tile into a ring of stages, each guarded by a "full"
//            mbarrier with a transaction count;
//   warp 1   allocates all 512 columns of tensor memory (two accumulators of BN columns), then one thread issues
//            tcgen05.mma.cta_group::1.kind::f16 (M = 128, N = BN, K = 16; four per k-block, operands described by
//            shared-memory matrix descriptors) and tcgen05.commit, which arrives on the stage's "empty" mbarrier when
//            the tensor core has read it, and on the accumulator's "ready" mbarrier after the tile's last k-block.
//            Tile i accumulates into accumulator i % 2, so its products run while the epilogue of tile i - 1 drains
//            the other one;
//   warps 2-5 epilogue: each reads its 32 lanes of the accumulator with tcgen05.ld (32 columns at a time), applies the
//            epilogue in float, rounds to bf16 once, stages boxes of 32 rows by 64 columns in shared memory for TMA
//            stores (cp.async.bulk.tensor, whole lines, clipped at the edges) and hands the accumulator back.
// Every wait on an mbarrier is bounded by a cycle count; a wait that runs out records error 5 and the block carries
// on to its end (tensor memory is always given back).  No cluster launch, no multicast.
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace cvb {

constexpr int kBM = 128;
constexpr int kBK = 64;                       // one 128-byte swizzle span of bf16
constexpr int kGemmThreads = 192;
constexpr int kBoxBytes = 32 * 64 * 2;        // what a warp of the epilogue hands to one TMA store: 32 rows of 64 bf16

enum GemmEpilogue { kPlain = 0, kSwiglu = 1, kAddResidual = 2 };

struct GemmParams {
    __nv_bfloat16* out;       // [M, n_out]
    const __nv_bfloat16* resid;   // [M, n_out] with kAddResidual (may be `out`)
    int M, N, K;              // N: rows of W
    int n_out;                // output columns: N, or N / 2 with SwiGLU
    int tiles_m, tiles_n, num_tiles;
    int* err;
};

// Tile t of the walk: groups of kGroupM row tiles are finished one after the other, and within a group the row tile runs
// fastest.  The blocks that run side by side then cover a patch of at most kGroupM row tiles by a few column tiles, whose
// activations and weight rows they share in the L2, however many rows the product has.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_origin(int t, const GemmParams& p, int out_cols, int& m0, int& n0) {
    const int per_group = kGroupM * p.tiles_n;
    const int group = t / per_group, r = t - group * per_group;
    const int rows = min(kGroupM, p.tiles_m - group * kGroupM);
    const int col = r / rows;
    m0 = (group * kGroupM + (r - col * rows)) * kBM;
    n0 = col * out_cols;
}

template <int BN, int STAGES>
struct GemmSmem {
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr size_t kBytes = 1024 + static_cast<size_t>(STAGES) * kStageBytes + 4 * 2 * kBoxBytes + (2 * STAGES + 4) * 8 + 16;
};

// kSwiglu: the B tile is 128 gate rows followed by the 128 matching up rows (BN must be 256); the output tile is
// 128 columns wide.  kAddResidual: out = rnd(rnd(A W^T) + resid), the sum the next layer's norm would otherwise make.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using L = GemmSmem<BN, STAGES>;
    constexpr bool SWIGLU = EPI == kSwiglu;
    static_assert(!SWIGLU || BN == 256, "gate and up rows share a tile of 256");
    pdl_trigger();
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* base = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    unsigned char* stages = base;
    unsigned char* staging = base + static_cast<size_t>(STAGES) * L::kStageBytes;      // 4 warps x 2 boxes, 1024-byte aligned
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + 4 * 2 * kBoxBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;              // [2]  tensor core: the tile's products are done
    uint64_t* acc_free = acc_ready + 2;                // [2]  128 epilogue threads: the accumulator has been read
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int OUT_COLS = SWIGLU ? BN / 2 : BN;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_ready + i, 1); mbar_init(acc_free + i, 128); }
        mbar_fence_init();
    }
    if (warp == 1) {                                   // one warp allocates both accumulators' columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                        // the activations come from the kernel before this one

    if (warp == 0) {
        if (lane == 0) {                               // ---- producer ----
            int it = 0;                                // k-blocks loaded so far, over all of this block's tiles
            for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
                int m0, n0;
                tile_origin(t, p, OUT_COLS, m0, n0);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES) mbar_wait(empty + s, ((it / STAGES) - 1) & 1, p.err);
                    unsigned char* a_dst = stages + static_cast<size_t>(s) * L::kStageBytes;
                    unsigned char* b_dst = a_dst + L::kABytes;
                    mbar_expect_tx(full + s, L::kStageBytes);
                    tma_load_2d(a_dst, &map_a, full + s, kb * kBK, m0);
                    tma_load_2d(b_dst, &map_w, full + s, kb * kBK, n0);
                    if constexpr (SWIGLU) tma_load_2d(b_dst + 128 * kBK * 2, &map_w, full + s, kb * kBK, p.n_out + n0);
                    else if constexpr (BN == 256) tma_load_2d(b_dst + 128 * kBK * 2, &map_w, full + s, kb * kBK, n0 + 128);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                               // ---- tensor-core issue ----
            constexpr uint32_t idesc = idesc_bf16(kBM, BN, false);
            int it = 0, i = 0;
            for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++i) {
                const int buf = i & 1, use = i >> 1;
                if (use > 0) {                         // the epilogue of the tile before last has drained this accumulator
                    mbar_wait(acc_free + buf, (use - 1) & 1, p.err);
                    tc_after();
                }
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    mbar_wait(full + s, (it / STAGES) & 1, p.err);
                    tc_after();
                    const uint32_t a_addr = smem_u32(stages + static_cast<size_t>(s) * L::kStageBytes);
                    const uint32_t b_addr = a_addr + L::kABytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        umma(tmem_d, desc_sw128(a_addr + k * 32, 16, 1024), desc_sw128(b_addr + k * 32, 16, 1024), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty + s);              // the stage is free once these products have read it
                }
                tc_commit(acc_ready + buf);
            }
        }
    } else {                                           // ---- epilogue: warps 2..5 own lanes 32 * (warp % 4) .. +31 ----
        // A warp turns 64 columns of its 32 rows into bf16, puts them into shared memory in the layout of a 128-byte
        // swizzled box (row r, 16-byte chunk j at chunk j ^ (r % 8)) and lets TMA store the box: whole lines, clipped
        // at the matrix's edges.  Two boxes per warp, so that one is stored while the next is filled.
        const int quarter = warp & 3;
        unsigned char* boxes = staging + (warp - 2) * (2 * kBoxBytes);
        int i = 0, n_box = 0;
        for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++i) {
            const int buf = i & 1, use = i >> 1;
            int m0, n0;
            tile_origin(t, p, OUT_COLS, m0, n0);
            const int row = m0 + quarter * 32 + lane;
            const uint32_t tmem_d = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
            mbar_wait(acc_ready + buf, use & 1, p.err);
            tc_after();
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 64, ++n_box) {
                if (n0 + c0 >= p.n_out) break;
                unsigned char* box = boxes + (n_box & 1) * kBoxBytes;
                if (lane == 0) bulk_wait_read<1>();    // the store before last, out of this box, has read it
                __syncwarp();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t v[32], u[32];
                    tm_load32(tmem_d + c0 + half * 32, v);
                    if constexpr (SWIGLU) tm_load32(tmem_d + OUT_COLS + c0 + half * 32, u);
                    tm_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 packed, old = make_uint4(0u, 0u, 0u, 0u);
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
                        if constexpr (EPI == kAddResidual) {
                            const int n = n0 + c0 + half * 32 + j;
                            if (row < p.M && n < p.n_out) old = *reinterpret_cast<const uint4*>(p.resid + static_cast<int64_t>(row) * p.n_out + n);
                        }
                        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float y0 = __uint_as_float(v[j + 2 * k]), y1 = __uint_as_float(v[j + 2 * k + 1]);
                            if constexpr (SWIGLU) {
                                const float g0 = rnd<__nv_bfloat16>(y0), g1 = rnd<__nv_bfloat16>(y1);
                                const float u0 = rnd<__nv_bfloat16>(__uint_as_float(u[j + 2 * k]));
                                const float u1 = rnd<__nv_bfloat16>(__uint_as_float(u[j + 2 * k + 1]));
                                y0 = rnd<__nv_bfloat16>(__fdividef(g0, 1.f + __expf(-g0))) * u0;
                                y1 = rnd<__nv_bfloat16>(__fdividef(g1, 1.f + __expf(-g1))) * u1;
                            }
                            if constexpr (EPI == kAddResidual) {
                                const float2 r = __bfloat1622float2(r2[k]);
                                y0 = rnd<__nv_bfloat16>(y0) + r.x;
                                y1 = rnd<__nv_bfloat16>(y1) + r.y;
                            }
                            h[k] = __floats2bfloat162_rn(y0, y1);
                        }
                        const int chunk = half * 4 + (j >> 3);
                        *reinterpret_cast<uint4*>(box + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = packed;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&map_out, box, n0 + c0, m0 + quarter * 32);
                    bulk_commit();
                }
            }
            tc_before();
            mbar_arrive(acc_free + buf);               // 128 arrivals: the next tile but one may overwrite it
        }
        if (lane == 0) bulk_wait<0>();                 // the stores are done before the block ends
    }
    tc_before();
    __syncthreads();
    if (warp == 1) {
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN));
    }
}

// ---- host side ------------------------------------------------------------------------------------------------

// Tensor map of a row-major bf16 matrix [rows, cols], fetched in boxes of [128 rows, 64 columns], 128-byte swizzle,
// zero fill outside the matrix.
static int matrix_map(CUtensorMap* out, const void* ptr, int64_t rows, int64_t cols) {
    return cached_bf16_map(out, ptr, rows, cols, kBK, 128);
}

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, int EPI>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, GemmParams p, cudaStream_t stream) {
    using L = GemmSmem<BN, STAGES>;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(L::kBytes));
        if (e != cudaSuccess) return static_cast<int>(e);
        set = true;
    }
    constexpr int OUT_COLS = EPI == kSwiglu ? BN / 2 : BN;
    p.tiles_m = (p.M + kBM - 1) / kBM;
    p.tiles_n = (p.n_out + OUT_COLS - 1) / OUT_COLS;
    const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    if (tiles > 2147483647LL) return CVB_E_SIZE;
    p.num_tiles = static_cast<int>(tiles);
    const unsigned blocks = static_cast<unsigned>(p.num_tiles < sm_count() ? p.num_tiles : sm_count());   // one per SM, persistent
    launch_kernel(gemm_tcgen05_kernel<BN, STAGES, EPI>, dim3(blocks), dim3(kGemmThreads), L::kBytes, stream, ma, mw, mo, p);
    return launch_status();
}

}  // namespace cvb

using namespace cvb;

// mode 0: C = A W^T.  mode 1: C = silu(A Wg^T) * (A Wu^T) with W = [Wg; Wu].  mode 2: C = rnd(A W^T) + resid (resid may
// be C itself).  tile_n: 128 or 256 (modes 0 and 2).
extern "C" int cvb_gemm_bf16_tcgen05(void* out, const void* a, const void* w, const void* resid, int M, int N, int K, int mode,
                                     int tile_n, int* err_flag, cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || N <= 0 || K <= 0) return CVB_E_SIZE;
    if (K % 8) return CVB_E_ALIGN;                     // rows of A and W must start on 16-byte boundaries for TMA
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(out) || !al(a) || !al(w) || !al(resid)) return CVB_E_ALIGN;
    if (mode == 1 && (N % 2)) return CVB_E_SHAPE;
    if (mode == 2 && !resid) return CVB_E_SHAPE;
    GemmParams p{};
    p.out = (__nv_bfloat16*)out; p.resid = (const __nv_bfloat16*)resid; p.M = M; p.N = N; p.K = K;
    p.n_out = mode == 1 ? N / 2 : N; p.err = err_flag;
    if (p.n_out % 8) return CVB_E_ALIGN;               // 16-byte stores of output rows
    CUtensorMap ma, mw, mo;
    int rc = matrix_map(&ma, a, M, K);
    if (rc != CVB_OK) return rc;
    rc = matrix_map(&mw, w, N, K);
    if (rc != CVB_OK) return rc;
    rc = cached_bf16_map(&mo, out, M, p.n_out, 64, 32);      // the epilogue stores boxes of 32 rows by 64 columns
    if (rc != CVB_OK) return rc;
    if (mode == 1) return launch_gemm<256, 4, kSwiglu>(ma, mw, mo, p, stream);
    if (mode == 0) return tile_n == 256 ? launch_gemm<256, 4, kPlain>(ma, mw, mo, p, stream) : launch_gemm<128, 6, kPlain>(ma, mw, mo, p, stream);
    if (mode == 2) return tile_n == 256 ? launch_gemm<256, 4, kAddResidual>(ma, mw, mo, p, stream) : launch_gemm<128, 6, kAddResidual>(ma, mw, mo, p, stream);
    return CVB_E_SHAPE;
}
