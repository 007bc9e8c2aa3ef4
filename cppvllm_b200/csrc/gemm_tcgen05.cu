// Matrix product on the fifth-generation tensor cores (tcgen05) for prompt portions, bf16:
//   C[M, N] = A[M, K] * W[N, K]^T          (A activations, W a weight matrix as checkpoints store it; both K-major)
// and its fused form for the gated feed-forward:
//   C[M, I] = T( rnd(silu(T(G))) * T(U) ),  G = A * W[0:I]^T,  U = A * W[I:2I]^T      (kernels/fused_ops.cu:210-220 of
//   the reference), where one tile's B operand is 128 gate rows over the 128 matching up rows, so that gate and up
//   of a column end up in the same accumulator row and the activations never travel through global memory.
//
// One block computes a 128 x BN tile (BN = 128 or 256).  Roles, by warp:
//   warp 0   producer: one thread issues TMA copies (cp.async.bulk.tensor.2d, 128-byte swizzle) of the A tile [128 x 64]
//            and the B tile [BN x 64] of every k-block into a ring of stages, each guarded by a "full" mbarrier with a
//            transaction count;
//   warp 1   allocates BN columns of tensor memory, then one thread issues tcgen05.mma.cta_group::1.kind::f16 (M = 128,
//            N = BN, K = 16; four per k-block, operands described by shared-memory matrix descriptors, accumulator in
//            tensor memory) and tcgen05.commit, which arrives on the stage's "empty" mbarrier when the tensor core has
//            read it, and on the "accumulator ready" mbarrier after the last k-block;
//   warps 2-5 epilogue: each reads its 32 lanes of the accumulator with tcgen05.ld (32 columns at a time), applies the
//            epilogue in float, rounds to bf16 once and stores rows to global memory.
// Every wait on an mbarrier is bounded by a cycle count; a wait that runs out records error 5 and the block carries
// on to its end (tensor memory is always given back).  No cluster launch, no multicast.
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace cvb {

constexpr int kBM = 128;
constexpr int kBK = 64;                       // one 128-byte swizzle span of bf16
constexpr int kGemmThreads = 192;

struct GemmParams {
    __nv_bfloat16* out;       // [M, n_out]
    int M, N, K;              // N: rows of W
    int n_out;                // output columns: N, or N / 2 with SwiGLU
    int* err;
};

template <int BN, int STAGES>
struct GemmSmem {
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr size_t kBytes = 1024 + static_cast<size_t>(STAGES) * kStageBytes + (2 * STAGES + 1) * 8 + 16;
};

// SWIGLU: the B tile is 128 gate rows followed by the 128 matching up rows (BN must be 256); the output tile is
// 128 columns wide.
template <int BN, int STAGES, bool SWIGLU>
__global__ void __launch_bounds__(kGemmThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using L = GemmSmem<BN, STAGES>;
    pdl_trigger();
    const uint32_t raw_addr = smem_u32(smem_raw);
    unsigned char* base = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    unsigned char* stages = base;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + static_cast<size_t>(STAGES) * L::kStageBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* accum_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_ready + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int OUT_COLS = SWIGLU ? BN / 2 : BN;
    const int m0 = blockIdx.y * kBM;
    const int n0 = blockIdx.x * OUT_COLS;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
        mbar_init(accum_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {                                   // one warp allocates the accumulator's columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem_d = *tmem_slot;
    pdl_wait();                                        // the activations come from the kernel before this one

    if (warp == 0) {
        if (lane == 0) {                               // ---- producer ----
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES) mbar_wait(empty + s, ((kb / STAGES) - 1) & 1, p.err);
                unsigned char* a_dst = stages + static_cast<size_t>(s) * L::kStageBytes;
                unsigned char* b_dst = a_dst + L::kABytes;
                mbar_expect_tx(full + s, L::kStageBytes);
                tma_load_2d(a_dst, &map_a, full + s, kb * kBK, m0);
                if constexpr (SWIGLU) {
                    tma_load_2d(b_dst, &map_w, full + s, kb * kBK, n0);
                    tma_load_2d(b_dst + 128 * kBK * 2, &map_w, full + s, kb * kBK, p.n_out + n0);
                } else {
                    tma_load_2d(b_dst, &map_w, full + s, kb * kBK, n0);
                    if constexpr (BN == 256) tma_load_2d(b_dst + 128 * kBK * 2, &map_w, full + s, kb * kBK, n0 + 128);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                               // ---- tensor-core issue ----
            constexpr uint32_t idesc = idesc_bf16(kBM, BN, false);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                mbar_wait(full + s, (kb / STAGES) & 1, p.err);
                tc_after();
                const uint32_t a_addr = smem_u32(stages + static_cast<size_t>(s) * L::kStageBytes);
                const uint32_t b_addr = a_addr + L::kABytes;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    umma(tmem_d, desc_sw128(a_addr + k * 32, 16, 1024), desc_sw128(b_addr + k * 32, 16, 1024), idesc,
                              (kb > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(empty + s);                // the stage is free once these products have read it
            }
            tc_commit(accum_ready);
        }
    } else {                                           // ---- epilogue: warps 2..5 own lanes 32 * (warp % 4) .. +31 ----
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        mbar_wait(accum_ready, 0, p.err);
        tc_after();
        __nv_bfloat16* out_row = p.out + static_cast<int64_t>(row) * p.n_out;
        for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
            uint32_t v[32], u[32];
            tm_load32(tmem_d + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
            if constexpr (SWIGLU) tm_load32(tmem_d + (static_cast<uint32_t>(quarter * 32) << 16) + OUT_COLS + c0, u);
            tm_wait_ld();
            if (row < p.M) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int n = n0 + c0 + j;
                    if (n >= p.n_out) break;
                    uint4 packed;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float y0 = __uint_as_float(v[j + 2 * i]), y1 = __uint_as_float(v[j + 2 * i + 1]);
                        if constexpr (SWIGLU) {
                            const float g0 = rnd<__nv_bfloat16>(y0), g1 = rnd<__nv_bfloat16>(y1);
                            const float u0 = rnd<__nv_bfloat16>(__uint_as_float(u[j + 2 * i]));
                            const float u1 = rnd<__nv_bfloat16>(__uint_as_float(u[j + 2 * i + 1]));
                            y0 = rnd<__nv_bfloat16>(g0 / (1.f + expf(-g0))) * u0;
                            y1 = rnd<__nv_bfloat16>(g1 / (1.f + expf(-g1))) * u1;
                        }
                        h[i] = __floats2bfloat162_rn(y0, y1);
                    }
                    if (n + 8 <= p.n_out) {
                        *reinterpret_cast<uint4*>(out_row + n) = packed;
                    } else {
                        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&packed);
                        for (int i = 0; n + i < p.n_out; ++i) out_row[n + i] = e[i];
                    }
                }
            }
        }
    }
    tc_before();
    __syncthreads();
    if (warp == 1) {
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(BN));
    }
}

// ---- host side ------------------------------------------------------------------------------------------------

// Tensor map of a row-major bf16 matrix [rows, cols], fetched in boxes of [128 rows, 64 columns], 128-byte swizzle,
// zero fill outside the matrix.
static int matrix_map(CUtensorMap* out, const void* ptr, int64_t rows, int64_t cols) {
    return cached_bf16_map(out, ptr, rows, cols, kBK, 128);
}

template <int BN, int STAGES, bool SWIGLU>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, const GemmParams& p, cudaStream_t stream) {
    using L = GemmSmem<BN, STAGES>;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(L::kBytes));
        if (e != cudaSuccess) return static_cast<int>(e);
        set = true;
    }
    constexpr int OUT_COLS = SWIGLU ? BN / 2 : BN;
    dim3 grid(static_cast<unsigned>((p.n_out + OUT_COLS - 1) / OUT_COLS), static_cast<unsigned>((p.M + kBM - 1) / kBM));
    launch_kernel(gemm_tcgen05_kernel<BN, STAGES, SWIGLU>, grid, dim3(kGemmThreads), L::kBytes, stream, ma, mw, p);
    return launch_status();
}

}  // namespace cvb

using namespace cvb;

// mode 0: C = A W^T.  mode 1: C = silu(A Wg^T) * (A Wu^T) with W = [Wg; Wu].  tile_n: 128 or 256 (mode 0 only).
extern "C" int cvb_gemm_bf16_tcgen05(void* out, const void* a, const void* w, int M, int N, int K, int mode, int tile_n,
                                     int* err_flag, cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || N <= 0 || K <= 0) return CVB_E_SIZE;
    if (K % 8) return CVB_E_ALIGN;                     // rows of A and W must start on 16-byte boundaries for TMA
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(out) || !al(a) || !al(w)) return CVB_E_ALIGN;
    if (mode == 1 && (N % 2)) return CVB_E_SHAPE;
    GemmParams p{};
    p.out = (__nv_bfloat16*)out; p.M = M; p.N = N; p.K = K; p.n_out = mode == 1 ? N / 2 : N; p.err = err_flag;
    if (p.n_out % 8) return CVB_E_ALIGN;               // 16-byte stores of output rows
    CUtensorMap ma, mw;
    int rc = matrix_map(&ma, a, M, K);
    if (rc != CVB_OK) return rc;
    rc = matrix_map(&mw, w, N, K);
    if (rc != CVB_OK) return rc;
    if (mode == 1) return launch_gemm<256, 4, true>(ma, mw, p, stream);
    if (mode != 0) return CVB_E_SHAPE;
    if (tile_n == 256) return launch_gemm<256, 4, false>(ma, mw, p, stream);
    return launch_gemm<128, 6, false>(ma, mw, p, stream);
}
