// Greedy and temperature sampling over float logits rows, one block per sampled row.
//
// Greedy (temperature <= 0): arg-max, ties to the lowest index (reference kernels/fused_ops.cu:303-304,339-340).
// Temperature: Gumbel-max, score_v = logit_v / max(temp, 1e-5) - log(max(-log u_v, 1e-10)) with
// u = ((x >> 8) + 0.5) / 2^24 from Philox4x32-10 (reference fused_ops.cu:287-309).  The reference feeds the
// generator with the row's index in the batch and a count of sampling calls (fused_ops.cu:330-335), so its
// tokens depend on what else was batched.  Here the key is the row's own 64-bit seed (derived on the host
// from the engine seed and the request) and the counter is (vocab index / 4, output position, tag, 0): a
// request's tokens are the same whatever it is batched with.
#include "common.cuh"

namespace cvb {

// Philox-4x32 with ten rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
struct Philox4 { uint32_t x, y, z, w; };
__device__ __forceinline__ Philox4 philox4x32_10(Philox4 ctr, uint32_t key_lo, uint32_t key_hi) {
    constexpr uint32_t kMulA = 0xD2511F53u, kMulB = 0xCD9E8D57u, kWeylA = 0x9E3779B9u, kWeylB = 0xBB67AE85u;
    for (int i = 0; i < 10; ++i) {
        Philox4 nxt;
        nxt.x = __umulhi(kMulB, ctr.z) ^ ctr.y ^ key_lo;
        nxt.y = kMulB * ctr.z;
        nxt.z = __umulhi(kMulA, ctr.x) ^ ctr.w ^ key_hi;
        nxt.w = kMulA * ctr.x;
        ctr = nxt;
        key_lo += kWeylA;
        key_hi += kWeylB;
    }
    return ctr;
}

__device__ __forceinline__ float uniform01(uint32_t x) {
    return (static_cast<float>(x >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct Best { float v; int i; };
__device__ __forceinline__ bool better(float v, int i, const Best& b) { return v > b.v || (v == b.v && i < b.i); }

constexpr uint32_t kSampleTag = 0x53414D50u;

__global__ void __launch_bounds__(1024)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, const int* __restrict__ rows,
              const float* __restrict__ temps, const uint64_t* __restrict__ seeds,
              const int* __restrict__ out_positions, int V, int n_logit_rows) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0) src = 0;
    if (src >= n_logit_rows) src = n_logit_rows - 1;
    const float* row = logits + static_cast<int64_t>(src) * V;
    const float temp = temps[r];
    const bool greedy = temp <= 0.f;
    const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
    const uint64_t seed = seeds[r];
    const uint32_t opos = static_cast<uint32_t>(out_positions[r]);

    Best best{-INFINITY, 0x7fffffff};
    for (int base = threadIdx.x * 4; base < V; base += blockDim.x * 4) {
        uint32_t rn[4] = {0, 0, 0, 0};
        if (!greedy) {
            const Philox4 g = philox4x32_10(Philox4{static_cast<uint32_t>(base >> 2), opos, kSampleTag, 0u},
                                            static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
            rn[0] = g.x; rn[1] = g.y; rn[2] = g.z; rn[3] = g.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (base + j >= V) break;
            const float x = row[base + j];
            float s = x;
            if (!greedy) {
                const float e = fmaxf(-logf(uniform01(rn[j])), 1e-10f);
                s = x * inv_t - logf(e);
            }
            if (better(s, base + j, best)) { best.v = s; best.i = base + j; }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, best.v, d);
        const int oi = __shfl_down_sync(0xffffffffu, best.i, d);
        if (better(ov, oi, best)) { best.v = ov; best.i = oi; }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
    __syncthreads();
    if (warp == 0) {
        best.v = lane < n_warps ? sv[lane] : -INFINITY;
        best.i = lane < n_warps ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_down_sync(0xffffffffu, best.v, d);
            const int oi = __shfl_down_sync(0xffffffffu, best.i, d);
            if (better(ov, oi, best)) { best.v = ov; best.i = oi; }
        }
        if (lane == 0) out[r] = best.i < V ? best.i : 0;   // a row of NaNs yields token 0, never an index >= V
    }
}

// Two-phase form for large vocabularies: phase 1 gives every row `n_chunks` blocks, each of which finds the best
// (score, index) of its slice of the vocabulary; phase 2 picks the best of a row's partial results.  Scores, random
// numbers and tie-breaking are those of sample_kernel, so both forms return the same token.
__global__ void __launch_bounds__(256)
sample_partial_kernel(float* __restrict__ part_v, int* __restrict__ part_i, const float* __restrict__ logits,
                      const int* __restrict__ rows, const float* __restrict__ temps, const uint64_t* __restrict__ seeds,
                      const int* __restrict__ out_positions, int V, int n_logit_rows, int n_chunks) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, chunk = blockIdx.y;
    int src = rows ? rows[r] : r;
    if (src < 0) src = 0;
    if (src >= n_logit_rows) src = n_logit_rows - 1;
    const float* row = logits + static_cast<int64_t>(src) * V;
    const float temp = temps[r];
    const bool greedy = temp <= 0.f;
    const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
    const uint64_t seed = seeds[r];
    const uint32_t opos = static_cast<uint32_t>(out_positions[r]);
    const int groups = (V + 3) >> 2;                                  // groups of four vocabulary entries
    const int per = (groups + n_chunks - 1) / n_chunks;
    const int g_begin = chunk * per, g_end = min(groups, g_begin + per);

    Best best{-INFINITY, 0x7fffffff};
    for (int gi = g_begin + threadIdx.x; gi < g_end; gi += blockDim.x) {
        const int base = gi << 2;
        uint32_t rn[4] = {0, 0, 0, 0};
        if (!greedy) {
            const Philox4 g = philox4x32_10(Philox4{static_cast<uint32_t>(gi), opos, kSampleTag, 0u},
                                            static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
            rn[0] = g.x; rn[1] = g.y; rn[2] = g.z; rn[3] = g.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (base + j >= V) break;
            const float x = row[base + j];
            float sc = x;
            if (!greedy) {
                const float e = fmaxf(-logf(uniform01(rn[j])), 1e-10f);
                sc = x * inv_t - logf(e);
            }
            if (better(sc, base + j, best)) { best.v = sc; best.i = base + j; }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, best.v, d);
        const int oi = __shfl_down_sync(0xffffffffu, best.i, d);
        if (better(ov, oi, best)) { best.v = ov; best.i = oi; }
    }
    __shared__ float sv[8];
    __shared__ int si[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w)
            if (better(sv[w], si[w], best)) { best.v = sv[w]; best.i = si[w]; }
        part_v[r * n_chunks + chunk] = best.v;
        part_i[r * n_chunks + chunk] = best.i;
    }
}

__global__ void sample_final_kernel(int* __restrict__ out, const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int V, int n_chunks) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    Best best{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const float v = part_v[r * n_chunks + c];
        const int i = part_i[r * n_chunks + c];
        if (better(v, i, best)) { best.v = v; best.i = i; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, best.v, d);
        const int oi = __shfl_down_sync(0xffffffffu, best.i, d);
        if (better(ov, oi, best)) { best.v = ov; best.i = oi; }
    }
    if (threadIdx.x == 0) out[r] = best.i < V ? best.i : 0;
}

// tokens[i] = sampled[src[i]] where src[i] >= 0: hands the previous step's samples to this step's inputs on
// the device (reference fused_ops.cu:380-397).
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                   const int* __restrict__ sampled, int n, int n_sampled) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int s = src[i];
    if (s >= 0 && s < n_sampled) tokens[i] = sampled[s];
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_sample(int* out, const float* logits, const int* rows, const float* temps,
                          const uint64_t* seeds, const int* out_positions, int R, int V, int n_logit_rows,
                          cudaStream_t stream) {
    if (R == 0) return CVB_OK;
    if (R < 0 || V <= 0 || n_logit_rows <= 0) return CVB_E_SIZE;
    launch_kernel(sample_kernel, dim3(R), dim3(1024), 0, stream, out, logits, rows, temps, seeds, out_positions, V, n_logit_rows);
    return launch_status();
}

// `scratch` holds R * n_chunks floats followed by R * n_chunks ints (n_chunks <= 64).
extern "C" int cvb_sample_chunked(int* out, const float* logits, const int* rows, const float* temps,
                                  const uint64_t* seeds, const int* out_positions, int R, int V, int n_logit_rows,
                                  int n_chunks, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    if (R == 0) return CVB_OK;
    if (R < 0 || V <= 0 || n_logit_rows <= 0 || n_chunks < 1 || n_chunks > 64) return CVB_E_SIZE;
    if (scratch == nullptr || scratch_bytes < static_cast<int64_t>(R) * n_chunks * 8) return CVB_E_SCRATCH;
    float* pv = static_cast<float*>(scratch);
    int* pi = reinterpret_cast<int*>(pv + static_cast<int64_t>(R) * n_chunks);
    dim3 grid(static_cast<unsigned>(R), static_cast<unsigned>(n_chunks));
    launch_kernel(sample_partial_kernel, dim3(grid), dim3(256), 0, stream, pv, pi, logits, rows, temps, seeds, out_positions, V, n_logit_rows, n_chunks);
    launch_kernel(sample_final_kernel, dim3(R), dim3(32), 0, stream, out, pv, pi, V, n_chunks);
    return launch_status();
}

extern "C" int cvb_feed_tokens(int* tokens, const int* src, const int* sampled, int n, int n_sampled,
                               cudaStream_t stream) {
    if (n == 0) return CVB_OK;
    if (n < 0) return CVB_E_SIZE;
    launch_kernel(feed_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, tokens, src, sampled, n, n_sampled);
    return launch_status();
}
