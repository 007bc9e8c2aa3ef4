// Two persistent kernels that carry a decode step of up to 8 tokens through a pre-norm block around its attention:
//
//   block head   h' = rnd(h + delta);  x = rmsnorm(h');  qkv = x Wqkv^T      | grid barrier |
//                per-head RMSNorm of q and k, rotary, q out, k and v into the cache pages
//   block tail   y1 = att Wo^T                                               | grid barrier |
//                h'' = rnd(h' + y1);  x = rmsnorm(h'');  act = swiglu(x Wgu^T)  | grid barrier |
//                y2 = act Wdown^T            (y2 is the next block's delta)
//
// Same arithmetic as the separate kernels (gemv_bf16.cu, qk_rope_kv.cu; formulas of the reference's
// kernels/fused_ops.cu:61-88, 104-207, 210-220).  What the fusion buys: a decode step is a chain of short products, each
// a few megabytes of weights; as separate kernels each pays its launch, its prologue and a first round trip to DRAM
// before its weights flow.  Here one block per SM stays resident and its weights arrive as ONE stream: the work of all
// phases is a list of rounds (one tile of a weight matrix per block and round); cp.async copies of the next three
// rounds are always in flight, each lane copying the 16-byte pieces it will itself feed to the tensor core into its own
// slots of a shared-memory ring.  Weights do not depend on the barriers, so the stream runs across them: while a block
// waits for the other blocks, or normalises its activations, the next phase's weights are already landing.
//
// The grid barrier is a counter and a generation word in global memory; the kernels are launched cooperatively, which
// guarantees that all blocks are resident.  Its spin is bounded by a cycle count: if it runs out the block records
// error 5 and goes on (the step's result is then discarded by the host).
#include "common.cuh"

namespace cvb {

constexpr int kFWarps = 8;
constexpr int kFThreads = kFWarps * 32;
constexpr int kFPad = 32;              // padding of activation rows in shared memory (elements)
constexpr int kFBatch = 8;             // rows of the step (columns of the B operand)

__device__ __forceinline__ void f_unpack8(const uint4& t, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ uint4 f_pack8(const float (&v)[8]) {
    uint4 t;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return t;
}
__device__ __forceinline__ void f_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- grid barrier (all blocks resident: cooperative launch) ---------------------------------------------------------
// bar[0] counts arrivals, bar[1] is the generation.  The last block to arrive bumps the generation; the others wait for
// the generation to change.
__device__ __forceinline__ void grid_barrier(unsigned int* bar, int* err) {
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int gen, arrived, now;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(gen) : "l"(bar + 1) : "memory");
        // the count wraps to zero with the last arrival, so nothing has to reset it; release: this block's writes (made
        // visible to this thread by the barrier above) are ordered before the arrival
        asm volatile("atom.acq_rel.gpu.global.inc.u32 %0, [%1], %2;\n" : "=r"(arrived) : "l"(bar), "r"(gridDim.x - 1) : "memory");
        if (arrived == gridDim.x - 1) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(bar + 1), "r"(gen + 1) : "memory");
        } else {
            const long long t0 = clock64();
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(now) : "l"(bar + 1) : "memory");
                if (now != gen) break;
                if (clock64() - t0 > 40000000LL) { atomicExch(err, 5); break; }
            }
        }
    }
    __syncthreads();
}

// ---- activations into shared memory ---------------------------------------------------------------------------------
// xs[m][K] = src[m][K] for m < M, zero rows above.  `src` may have been written by other blocks in an earlier phase:
// it is read past L1.
__device__ __forceinline__ void stage_copy(__nv_bfloat16* xs, const __nv_bfloat16* src, int M, int K) {
    const int chunks = K >> 3, xstride = K + kFPad;
    const int total = kFBatch * chunks;
    for (int i0 = threadIdx.x; i0 < total; i0 += kFThreads * 8) {       // eight loads in flight per thread
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * kFThreads;
            const int m = i / chunks, c = i - m * chunks;
            v[u] = (i < total && m < M) ? __ldcg(reinterpret_cast<const uint4*>(src + static_cast<int64_t>(m) * K + c * 8)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * kFThreads;
            if (i < total) { const int m = i / chunks, c = i - m * chunks; *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = v[u]; }
        }
    }
}

// The residual stream is known when the kernel starts: it can be parked in shared memory (`hs`, same layout as xs)
// before a barrier, so that only the delta has to be fetched after it.
__device__ __forceinline__ void park_rows(__nv_bfloat16* hs, const __nv_bfloat16* h, int M, int K) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = K >> 3, xstride = K + kFPad;
    for (int m = warp; m < M; m += kFWarps)
        for (int c = lane; c < chunks; c += 32)
            *reinterpret_cast<uint4*>(hs + m * xstride + c * 8) = __ldcg(reinterpret_cast<const uint4*>(h + static_cast<int64_t>(m) * K + c * 8));
}

// xs = rmsnorm(rnd(h + delta)) * w, one warp per row; block 0 writes the new residual stream to h_out.  With `hs`,
// h is read from there (park_rows put it there, the same lanes read it back); `w` may point into shared memory.
__device__ __forceinline__ void stage_norm(__nv_bfloat16* xs, const __nv_bfloat16* h, const __nv_bfloat16* delta,
                                           __nv_bfloat16* h_out, const float* w, float eps, int M, int K,
                                           const __nv_bfloat16* hs = nullptr) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = K >> 3, xstride = K + kFPad;
    for (int m = warp; m < kFBatch; m += kFWarps) {
        if (m >= M) {
            for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = make_uint4(0, 0, 0, 0);
            continue;
        }
        float ss = 0.f;
        for (int c = lane; c < chunks; c += 32) {
            float v[8];
            if (hs != nullptr) f_unpack8(*reinterpret_cast<const uint4*>(hs + m * xstride + c * 8), v);
            else f_unpack8(__ldcg(reinterpret_cast<const uint4*>(h + static_cast<int64_t>(m) * K + c * 8)), v);
            if (delta != nullptr) {
                float d[8];
                f_unpack8(__ldcg(reinterpret_cast<const uint4*>(delta + static_cast<int64_t>(m) * K + c * 8)), d);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = rnd<__nv_bfloat16>(v[i] + d[i]);
            }
            const uint4 packed = f_pack8(v);
            *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = packed;
            if (delta != nullptr && blockIdx.x == 0)
                *reinterpret_cast<uint4*>(h_out + static_cast<int64_t>(m) * K + c * 8) = packed;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(K) + eps);
        for (int c = lane; c < chunks; c += 32) {                  // each lane re-reads the chunks it wrote itself
            float v[8];
            f_unpack8(*reinterpret_cast<const uint4*>(xs + m * xstride + c * 8), v);
            const float4 w0 = *reinterpret_cast<const float4*>(w + c * 8);
            const float4 w1 = *reinterpret_cast<const float4*>(w + c * 8 + 4);
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = rnd<__nv_bfloat16>(v[i] * inv) * ww[i];
            *reinterpret_cast<uint4*>(xs + m * xstride + c * 8) = f_pack8(v);
        }
    }
}

// ---- the weight stream ----------------------------------------------------------------------------------------------------
// A phase is a product out[m, n] = sum_k xs[m, k] W[n, k].  Its tiles (16 rows of W, or 8 with the lower half of the A
// operand left zero, or 8 gate rows over the 8 matching up rows) go round-robin to the blocks: round i of a phase is tile
// blockIdx.x + i * gridDim.x.  The eight warps of a block split K.
struct PhaseDesc {
    const __nv_bfloat16* W;
    int N, K;                 // rows and columns of W
    int tile_rows;            // 8 or 16
    int swiglu;               // 1: tile = 8 gate rows over the 8 matching up rows, output silu(gate) * up
    int n_out, n_tiles, rounds, per_warp;   // derived
};

__device__ __forceinline__ PhaseDesc make_phase(const __nv_bfloat16* W, int N, int K, int tile_rows, int swiglu) {
    PhaseDesc d;
    d.W = W; d.N = N; d.K = K; d.tile_rows = tile_rows; d.swiglu = swiglu;
    d.n_out = swiglu ? N / 2 : N;
    const int out_per_tile = swiglu ? 8 : tile_rows;
    d.n_tiles = (d.n_out + out_per_tile - 1) / out_per_tile;
    d.rounds = (d.n_tiles + gridDim.x - 1) / gridDim.x;
    d.per_warp = (((K + 31) >> 5) + kFWarps - 1) / kFWarps;
    return d;
}

constexpr int kRing = 3;               // rounds in flight

__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem), "r"(n));
}

// Copies this thread's pieces of one round into its slots: piece (u, half) of thread t sits at
// slot[(u * halves + half) * 256 + t], halves = 2 for tiles with a lower half, else 1.
__device__ __forceinline__ void issue_round(const PhaseDesc& d, int round, uint4* slot) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
    const int tile = blockIdx.x + round * gridDim.x;
    const int out_per_tile = d.swiglu ? 8 : d.tile_rows;
    const int n0 = tile * out_per_tile;
    const bool tile_ok = round < d.rounds && tile < d.n_tiles;
    const bool lower = d.swiglu || d.tile_rows == 16;
    const int chunks = d.K >> 3, slabs = (d.K + 31) >> 5;
    const int j_begin = warp * d.per_warp, j_end = min(slabs, j_begin + d.per_warp);
    const int row_hi = min(n0 + r, d.N - 1);
    const int row_lo = min(d.swiglu ? d.n_out + n0 + r : n0 + r + 8, d.N - 1);
    const uint4* w_hi = reinterpret_cast<const uint4*>(d.W + static_cast<int64_t>(row_hi) * d.K);
    const uint4* w_lo = reinterpret_cast<const uint4*>(d.W + static_cast<int64_t>(row_lo) * d.K);
    for (int u = 0; u < d.per_warp; ++u) {
        const int c = (j_begin + u) * 4 + q;
        const bool ok = tile_ok && j_begin + u < j_end && c < chunks;
        const int halves = lower ? 2 : 1;
        cp16(slot + (u * halves) * kFThreads + threadIdx.x, ok ? static_cast<const void*>(w_hi + c) : static_cast<const void*>(d.W), ok);
        if (lower) cp16(slot + (u * 2 + 1) * kFThreads + threadIdx.x, ok ? static_cast<const void*>(w_lo + c) : static_cast<const void*>(d.W), ok);
    }
}

// The stream: a flat list of rounds over up to three phases, issued kRing rounds ahead of their use.
struct Stream {
    PhaseDesc ph[3];
    int n_phases;
    int issued;               // rounds issued so far (flat index)
    uint4* ring;              // kRing slots of slot_elems uint4 each
    int slot_elems;

    __device__ __forceinline__ void issue_next() {            // always commits a group, possibly an empty one
        int i = issued, p = 0;
        while (p < n_phases && i >= ph[p].rounds) { i -= ph[p].rounds; ++p; }
        if (p < n_phases) issue_round(ph[p], i, ring + (issued % kRing) * slot_elems);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        ++issued;
    }
};

// Runs one phase: for each of its rounds waits for the round's weights, multiplies, adds the warps' parts and stores.
// `first_flat` is the flat index of the phase's first round.
__device__ __forceinline__ void run_phase(Stream& st, int p, int first_flat, const __nv_bfloat16* xs, float* red,
                                          __nv_bfloat16* out, int M) {
    const PhaseDesc& d = st.ph[p];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
    const int chunks = d.K >> 3, slabs = (d.K + 31) >> 5, xstride = d.K + kFPad;
    const int j_begin = warp * d.per_warp, j_end = min(slabs, j_begin + d.per_warp);
    const uint4* x_row = reinterpret_cast<const uint4*>(xs + r * xstride);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const bool lower = d.swiglu || d.tile_rows == 16;
    const int out_per_tile = d.swiglu ? 8 : d.tile_rows;
    for (int round = 0; round < d.rounds; ++round) {
        // rounds first_flat + round + 1 .. + kRing - 1 may still be in flight
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kRing - 1) : "memory");
        const uint4* slot = st.ring + ((first_flat + round) % kRing) * st.slot_elems;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int u = 0; u < d.per_warp; ++u) {
            if (j_begin + u >= j_end) break;
            const int c = (j_begin + u) * 4 + q;
            const uint4 hi = slot[(u * (lower ? 2 : 1)) * kFThreads + threadIdx.x];
            const uint4 lo = lower ? slot[(u * 2 + 1) * kFThreads + threadIdx.x] : zero;
            const uint4 xv = c < chunks ? x_row[c] : zero;
            f_mma(acc, hi.x, lo.x, hi.y, lo.y, xv.x, xv.y);
            f_mma(acc, hi.z, lo.z, hi.w, lo.w, xv.z, xv.w);
        }
        float* mine = red + warp * 128;
        mine[r * 8 + 2 * q] = acc[0];
        mine[r * 8 + 2 * q + 1] = acc[1];
        mine[(r + 8) * 8 + 2 * q] = acc[2];
        mine[(r + 8) * 8 + 2 * q + 1] = acc[3];
        __syncthreads();                                       // all warps have read this round's slot
        st.issue_next();                                       // refill it with the round kRing ahead
        const int tile = blockIdx.x + round * gridDim.x;
        if (threadIdx.x < out_per_tile * kFBatch && tile < d.n_tiles) {
            const int row = threadIdx.x / kFBatch, m = threadIdx.x % kFBatch;
            const int n = tile * out_per_tile + row;
            if (n < d.n_out && m < M) {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int w = 0; w < kFWarps; ++w) {
                    s0 += red[w * 128 + row * 8 + m];
                    if (d.swiglu) s1 += red[w * 128 + (row + 8) * 8 + m];
                }
                float y = s0;
                if (d.swiglu) {
                    const float g = rnd<__nv_bfloat16>(s0), u = rnd<__nv_bfloat16>(s1);
                    y = rnd<__nv_bfloat16>(g / (1.f + expf(-g))) * u;
                }
                out[static_cast<int64_t>(m) * d.n_out + n] = __float2bfloat16_rn(y);
            }
        }
        __syncthreads();                                       // `red` is free again
    }
}

// ---- block tail ---------------------------------------------------------------------------------------------------------

struct TailParams {
    const __nv_bfloat16* att;      // [M, Kq]
    const __nv_bfloat16* w_o;      // [D, Kq]
    __nv_bfloat16* y1;             // [M, D]
    const __nv_bfloat16* h_in;     // [M, D]
    __nv_bfloat16* h_out;          // [M, D]
    const float* norm_w;           // [D]
    const __nv_bfloat16* w_gu;     // [2I, D]
    __nv_bfloat16* act;            // [M, I]
    const __nv_bfloat16* w_down;   // [D, I]
    __nv_bfloat16* y2;             // [M, D]
    int M, D, Kq, I;
    int slot_elems;                // uint4 per ring slot
    float eps;
    unsigned int* barrier;
    int* err;
};

__device__ __forceinline__ int small_n_tile_rows(int n) { return n / 16 >= 120 ? 16 : 8; }

__global__ void __launch_bounds__(kFThreads)
decode_block_tail_kernel(const TailParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const int kmax = max(max(p.Kq, p.D), p.I);
    float* red = reinterpret_cast<float*>(xs + kFBatch * (kmax + kFPad));
    Stream st;
    st.ring = reinterpret_cast<uint4*>(red + kFWarps * 128);
    st.slot_elems = p.slot_elems;
    st.n_phases = 3;
    st.issued = 0;
    st.ph[0] = make_phase(p.w_o, p.D, p.Kq, small_n_tile_rows(p.D), 0);
    st.ph[1] = make_phase(p.w_gu, 2 * p.I, p.D, 16, 1);
    st.ph[2] = make_phase(p.w_down, p.D, p.I, small_n_tile_rows(p.D), 0);
    __nv_bfloat16* hs = reinterpret_cast<__nv_bfloat16*>(st.ring + kRing * p.slot_elems);
    float* ws = reinterpret_cast<float*>(hs + kFBatch * (p.D + kFPad));
    pdl_trigger();
    for (int i = 0; i < kRing; ++i) st.issue_next();               // weights do not depend on earlier kernels
    for (int i = threadIdx.x; i < p.D; i += kFThreads) ws[i] = p.norm_w[i];
    pdl_wait();
    stage_copy(xs, p.att, p.M, p.Kq);
    park_rows(hs, p.h_in, p.M, p.D);                               // known already: only y1 is fetched after the barrier
    __syncthreads();
    run_phase(st, 0, 0, xs, red, p.y1, p.M);
    grid_barrier(p.barrier, p.err);
    stage_norm(xs, p.h_in, p.y1, p.h_out, ws, p.eps, p.M, p.D, hs);
    __syncthreads();
    run_phase(st, 1, st.ph[0].rounds, xs, red, p.act, p.M);
    grid_barrier(p.barrier, p.err);
    stage_copy(xs, p.act, p.M, p.I);
    __syncthreads();
    run_phase(st, 2, st.ph[0].rounds + st.ph[1].rounds, xs, red, p.y2, p.M);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

// ---- block head ---------------------------------------------------------------------------------------------------------

struct HeadParams {
    const __nv_bfloat16* h_in;     // [M, D]
    const __nv_bfloat16* delta;    // [M, D] or nullptr
    __nv_bfloat16* h_out;          // [M, D] (used when delta is given)
    const float* norm_w;           // [D]
    const __nv_bfloat16* w_qkv;    // [(H + 2 KV) hd, D]
    __nv_bfloat16* qkv;            // [M, (H + 2 KV) hd]
    __nv_bfloat16* q_out;          // [M, H, hd]
    const float* q_w;              // per-head norm weights or nullptr
    const float* k_w;
    const float* cos_t;            // [max_pos, hd / 2] or nullptr
    const float* sin_t;
    const int* positions;          // [M]
    const int* slots;              // [M]
    __nv_bfloat16* cache;          // [pages, 2, KV, page, hd]
    int M, D, H, KV, hd, page_size, max_pos;
    int slot_elems;
    int64_t cache_elems;
    float eps, qk_eps;
    unsigned int* barrier;
    int* err;
};

__global__ void __launch_bounds__(kFThreads)
decode_block_head_kernel(const HeadParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* red = reinterpret_cast<float*>(xs + kFBatch * (p.D + kFPad));
    const int N = (p.H + 2 * p.KV) * p.hd;
    Stream st;
    st.ring = reinterpret_cast<uint4*>(red + kFWarps * 128);
    st.slot_elems = p.slot_elems;
    st.n_phases = 1;
    st.issued = 0;
    st.ph[0] = make_phase(p.w_qkv, N, p.D, small_n_tile_rows(N), 0);
    float* ws = reinterpret_cast<float*>(st.ring + kRing * p.slot_elems);
    pdl_trigger();
    for (int i = 0; i < kRing; ++i) st.issue_next();
    for (int i = threadIdx.x; i < p.D; i += kFThreads) ws[i] = p.norm_w[i];
    pdl_wait();
    __syncthreads();
    stage_norm(xs, p.h_in, p.delta, p.h_out, ws, p.eps, p.M, p.D);
    __syncthreads();
    run_phase(st, 0, 0, xs, red, p.qkv, p.M);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    grid_barrier(p.barrier, p.err);

    // per-head norm, rotary, cache write: hd / 8 neighbouring lanes own one head vector (16-byte chunks)
    const int CH = p.hd >> 3;                                      // a power of two between 2 and 32 (checked on the host)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_warp = 32 / CH;
    const int n_tasks = p.H + 2 * p.KV;
    const int items = p.M * n_tasks;
    const int c = lane % CH;
    for (int base = (blockIdx.x * kFWarps + warp) * per_warp; base < items; base += gridDim.x * kFWarps * per_warp) {
        const int item = base + lane / CH;
        const bool active = item < items;
        const int m = active ? item / n_tasks : 0, task = active ? item % n_tasks : 0;
        const bool is_q = task < p.H, is_v = task >= p.H + p.KV;
        const int slot = p.slots[m];
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = 0.f;
        if (active) f_unpack8(__ldcg(reinterpret_cast<const uint4*>(p.qkv + (static_cast<int64_t>(m) * n_tasks + task) * p.hd + c * 8)), x);
        __nv_bfloat16* dst = nullptr;
        if (active) {
            if (is_q) {
                dst = p.q_out + (static_cast<int64_t>(m) * p.H + task) * p.hd + c * 8;
            } else if (slot >= 0) {
                const int kvh = is_v ? task - p.H - p.KV : task - p.H;
                const int64_t page = slot / p.page_size, off = slot % p.page_size;
                const int64_t b = (((page * 2 + (is_v ? 1 : 0)) * p.KV + kvh) * p.page_size + off) * p.hd;
                if (b + p.hd > p.cache_elems) { if (c == 0) atomicExch(p.err, 2); }
                else dst = p.cache + b + c * 8;
            }
        }
        if (active && is_v && dst != nullptr) *reinterpret_cast<uint4*>(dst) = f_pack8(x);
        const float* w = is_q ? p.q_w : p.k_w;
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
        for (int o = CH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (w != nullptr && active && !is_v) {
            const float inv = rsqrtf(ss / static_cast<float>(p.hd) + p.qk_eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = rnd<__nv_bfloat16>(rnd<__nv_bfloat16>(x[i] * inv) * w[c * 8 + i]);
        }
        float other[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, x[i], CH >> 1);
        if (!active || is_v || dst == nullptr) continue;
        if (p.cos_t != nullptr) {
            int pos = p.positions[m];
            if (pos < 0 || pos >= p.max_pos) {
                if (c == 0) atomicExch(p.err, 3);
                pos = pos < 0 ? 0 : p.max_pos - 1;
            }
            const bool first = c < (CH >> 1);
            const int e0 = (first ? c : c - (CH >> 1)) * 8;
            const float* cr = p.cos_t + static_cast<int64_t>(pos) * (p.hd >> 1) + e0;
            const float* sr = p.sin_t + static_cast<int64_t>(pos) * (p.hd >> 1) + e0;
            float o8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o8[i] = first ? x[i] * cr[i] - other[i] * sr[i] : x[i] * cr[i] + other[i] * sr[i];
            *reinterpret_cast<uint4*>(dst) = f_pack8(o8);
        } else {
            *reinterpret_cast<uint4*>(dst) = f_pack8(x);
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------------

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

template <typename P>
static int launch_cooperative(void (*kernel)(P), const P& p, size_t smem, cudaStream_t stream) {
    if (smem > 220 * 1024) return CVB_E_SIZE;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kFThreads, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (per_sm < 1) return CVB_E_SIZE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count()));       // one block per SM: all resident, as the barrier needs
    cfg.blockDim = dim3(kFThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, p);
    return e == cudaSuccess ? launch_status() : static_cast<int>(e);
}

static bool aligned16(const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; }
static int per_warp_slabs(int K) { return (((K + 31) / 32) + kFWarps - 1) / kFWarps; }
static int tile_rows_for(int n) { return n / 16 >= 120 ? 16 : 8; }

}  // namespace cvb

using namespace cvb;

// `barrier`: two unsigned ints in device memory, zero when first used; the kernels leave the count at zero.
extern "C" int cvb_decode_block_tail(const void* att, const void* w_o, void* y1, const void* h_in, void* h_out,
                                     const float* norm_w, const void* w_gu, void* act, const void* w_down, void* y2,
                                     int M, int D, int Kq, int I, float eps, unsigned int* barrier, int* err_flag,
                                     cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || M > kFBatch || D <= 0 || Kq <= 0 || I <= 0) return CVB_E_SIZE;
    if ((D % 8) || (Kq % 8) || (I % 8)) return CVB_E_ALIGN;
    if (!aligned16(att) || !aligned16(w_o) || !aligned16(y1) || !aligned16(h_in) || !aligned16(h_out) || !aligned16(norm_w) ||
        !aligned16(w_gu) || !aligned16(act) || !aligned16(w_down) || !aligned16(y2))
        return CVB_E_ALIGN;
    if (barrier == nullptr || h_out == h_in) return CVB_E_SHAPE;
    TailParams p{};
    p.att = (const __nv_bfloat16*)att; p.w_o = (const __nv_bfloat16*)w_o; p.y1 = (__nv_bfloat16*)y1;
    p.h_in = (const __nv_bfloat16*)h_in; p.h_out = (__nv_bfloat16*)h_out; p.norm_w = norm_w;
    p.w_gu = (const __nv_bfloat16*)w_gu; p.act = (__nv_bfloat16*)act; p.w_down = (const __nv_bfloat16*)w_down;
    p.y2 = (__nv_bfloat16*)y2; p.M = M; p.D = D; p.Kq = Kq; p.I = I; p.eps = eps; p.barrier = barrier; p.err = err_flag;
    const int kmax = Kq > D ? (Kq > I ? Kq : I) : (D > I ? D : I);
    // a ring slot holds one round of the widest phase: per thread per_warp pieces, twice that for 16-row tiles
    const int pieces_o = per_warp_slabs(Kq) * (tile_rows_for(D) == 16 ? 2 : 1);
    const int pieces_gu = per_warp_slabs(D) * 2;
    const int pieces_down = per_warp_slabs(I) * (tile_rows_for(D) == 16 ? 2 : 1);
    const int pieces = pieces_o > pieces_gu ? (pieces_o > pieces_down ? pieces_o : pieces_down) : (pieces_gu > pieces_down ? pieces_gu : pieces_down);
    p.slot_elems = pieces * kFThreads;
    const size_t smem = static_cast<size_t>(kFBatch) * (kmax + kFPad) * sizeof(__nv_bfloat16) + kFWarps * 128 * sizeof(float) +
                        static_cast<size_t>(kRing) * p.slot_elems * sizeof(uint4) +
                        static_cast<size_t>(kFBatch) * (D + kFPad) * sizeof(__nv_bfloat16) + static_cast<size_t>(D) * sizeof(float);
    return launch_cooperative(decode_block_tail_kernel, p, smem, stream);
}

extern "C" int cvb_decode_block_head(const void* h_in, const void* delta, void* h_out, const float* norm_w,
                                     const void* w_qkv, void* qkv, void* q_out, const float* q_w, const float* k_w,
                                     const float* cos_t, const float* sin_t, const int* positions, const int* slots,
                                     void* cache, int M, int D, int H, int KV, int hd, int page_size, int max_pos,
                                     int64_t cache_elems, float eps, float qk_eps, unsigned int* barrier,
                                     int* err_flag, cudaStream_t stream) {
    if (M == 0) return CVB_OK;
    if (M < 0 || M > kFBatch || D <= 0 || H <= 0 || KV <= 0 || hd <= 0 || page_size <= 0) return CVB_E_SIZE;
    if (D % 8) return CVB_E_ALIGN;
    const int CH = hd / 8;
    if (hd % 8 || CH < 2 || CH > 32 || (CH & (CH - 1))) return CVB_E_UNSUPPORTED;
    if ((q_w == nullptr) != (k_w == nullptr)) return CVB_E_SHAPE;
    if (cos_t != nullptr && (sin_t == nullptr || positions == nullptr || max_pos <= 0)) return CVB_E_SHAPE;
    if (!aligned16(h_in) || !aligned16(delta) || !aligned16(h_out) || !aligned16(norm_w) || !aligned16(w_qkv) || !aligned16(qkv) ||
        !aligned16(q_out) || !aligned16(cache) || !aligned16(cos_t) || !aligned16(sin_t))
        return CVB_E_ALIGN;
    if (barrier == nullptr || slots == nullptr || cache == nullptr) return CVB_E_SHAPE;
    if (delta != nullptr && (h_out == nullptr || h_out == h_in)) return CVB_E_SHAPE;
    HeadParams p{};
    p.h_in = (const __nv_bfloat16*)h_in; p.delta = (const __nv_bfloat16*)delta; p.h_out = (__nv_bfloat16*)h_out;
    p.norm_w = norm_w; p.w_qkv = (const __nv_bfloat16*)w_qkv; p.qkv = (__nv_bfloat16*)qkv; p.q_out = (__nv_bfloat16*)q_out;
    p.q_w = q_w; p.k_w = k_w; p.cos_t = cos_t; p.sin_t = sin_t; p.positions = positions; p.slots = slots;
    p.cache = (__nv_bfloat16*)cache; p.M = M; p.D = D; p.H = H; p.KV = KV; p.hd = hd; p.page_size = page_size;
    p.max_pos = max_pos; p.cache_elems = cache_elems; p.eps = eps; p.qk_eps = qk_eps; p.barrier = barrier; p.err = err_flag;
    const int N = (H + 2 * KV) * hd;
    p.slot_elems = per_warp_slabs(D) * (tile_rows_for(N) == 16 ? 2 : 1) * kFThreads;
    const size_t smem = static_cast<size_t>(kFBatch) * (D + kFPad) * sizeof(__nv_bfloat16) + kFWarps * 128 * sizeof(float) +
                        static_cast<size_t>(kRing) * p.slot_elems * sizeof(uint4) + static_cast<size_t>(D) * sizeof(float);
    return launch_cooperative(decode_block_head_kernel, p, smem, stream);
}
