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

constexpr uint32_t kSampleTag = 0x53414D50u;

// A candidate (score, vocabulary index) as one 64-bit word whose unsigned order is the sampler's order: the higher
// score wins, among equal scores the lower index.  0 stands for "no candidate"; a NaN score is no candidate.
__device__ __forceinline__ unsigned long long candidate(float score, int index) {
    if (score != score) return 0ull;
    uint32_t bits = __float_as_uint(score);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);          // floats in their order, as unsigned numbers
    return (static_cast<unsigned long long>(bits) << 32) | static_cast<uint32_t>(0x7fffffff - index);
}
__device__ __forceinline__ int candidate_token(unsigned long long c, int V) {
    const int index = 0x7fffffff - static_cast<int>(static_cast<uint32_t>(c));
    return (c != 0ull && index >= 0 && index < V) ? index : 0;           // a row of NaNs yields token 0, never an index >= V
}
__device__ __forceinline__ unsigned long long best_of_warp(unsigned long long c) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, c, o);
        c = other > c ? other : c;
    }
    return c;
}

// What a sampled row needs, read once per block.
struct RowDraw {
    const float* logits;
    float inv_temp;
    bool greedy, vec4;
    uint32_t key_lo, key_hi, out_pos;
};
__device__ __forceinline__ RowDraw row_draw(int r, const float* logits, const int* rows, const float* temps,
                                            const uint64_t* seeds, const int* out_positions, int V, int n_logit_rows) {
    int src = rows != nullptr ? rows[r] : r;
    src = max(0, min(src, n_logit_rows - 1));
    const float temp = temps[r];
    const uint64_t seed = seeds[r];
    const float* row = logits + static_cast<int64_t>(src) * V;
    return RowDraw{row, 1.0f / fmaxf(temp, 1e-5f), temp <= 0.f, (reinterpret_cast<uintptr_t>(row) & 15) == 0,
                   static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), static_cast<uint32_t>(out_positions[r])};
}

// The best candidate among the groups of four vocabulary entries g_begin + threadIdx.x, + blockDim.x, ... below g_end.
// One Philox call serves a group; the counter names the group, so a score does not depend on who computes it.
__device__ __forceinline__ unsigned long long best_of_groups(const RowDraw& d, int V, int g_begin, int g_end) {
    unsigned long long best = 0ull;
    for (int group = g_begin + threadIdx.x; group < g_end; group += blockDim.x) {
        uint32_t bits[4] = {0u, 0u, 0u, 0u};
        if (!d.greedy) {
            const Philox4 p = philox4x32_10(Philox4{static_cast<uint32_t>(group), d.out_pos, kSampleTag, 0u}, d.key_lo, d.key_hi);
            bits[0] = p.x; bits[1] = p.y; bits[2] = p.z; bits[3] = p.w;
        }
        const int first = group << 2, n = min(4, V - first);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (d.vec4 && n == 4) {                               // the row starts on a 16-byte boundary: one load a group
            const float4 q = __ldcs(reinterpret_cast<const float4*>(d.logits + first));
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
            for (int j = 0; j < n; ++j) v[j] = d.logits[first + j];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j >= n) break;
            float score = v[j];
            if (!d.greedy) score = score * d.inv_temp - logf(fmaxf(-logf(uniform01(bits[j])), 1e-10f));   // Gumbel-max
            const unsigned long long c = candidate(score, first + j);
            best = c > best ? c : best;
        }
    }
    return best;
}

// Grid (rows, chunks): block (r, chunk) searches its share of row r's vocabulary.  With one chunk the block writes
// the token; with more it leaves its best candidate in `part[r * n_chunks + chunk]` for sample_pick_kernel.  Either
// way a row's token is the largest candidate over the whole vocabulary, so every chunk count gives the same token.
__global__ void __launch_bounds__(1024)
sample_search_kernel(int* __restrict__ out, unsigned long long* __restrict__ part, const float* __restrict__ logits,
                     const int* __restrict__ rows, const float* __restrict__ temps, const uint64_t* __restrict__ seeds,
                     const int* __restrict__ out_positions, int V, int n_logit_rows, int n_chunks) {
    pdl_trigger();
    pdl_wait();
    __shared__ unsigned long long per_warp[32];
    const int r = blockIdx.x, chunk = blockIdx.y;
    const RowDraw d = row_draw(r, logits, rows, temps, seeds, out_positions, V, n_logit_rows);
    const int groups = (V + 3) >> 2;
    const int share = (groups + n_chunks - 1) / n_chunks;
    unsigned long long best = best_of_warp(best_of_groups(d, V, chunk * share, min(groups, (chunk + 1) * share)));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    if (lane == 0) per_warp[warp] = best;
    __syncthreads();
    if (warp != 0) return;
    best = best_of_warp(lane < n_warps ? per_warp[lane] : 0ull);
    if (lane != 0) return;
    if (n_chunks == 1) out[r] = candidate_token(best, V);
    else part[static_cast<int64_t>(r) * n_chunks + chunk] = best;
}

__global__ void sample_pick_kernel(int* __restrict__ out, const unsigned long long* __restrict__ part, int V, int n_chunks) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    unsigned long long best = 0ull;
    for (int c = threadIdx.x; c < n_chunks; c += 32) {
        const unsigned long long other = part[static_cast<int64_t>(r) * n_chunks + c];
        best = other > best ? other : best;
    }
    best = best_of_warp(best);
    if (threadIdx.x == 0) out[r] = candidate_token(best, V);
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
    launch_kernel(sample_search_kernel, dim3(R), dim3(1024), 0, stream, out, static_cast<unsigned long long*>(nullptr), logits, rows,
                  temps, seeds, out_positions, V, n_logit_rows, 1);
    return launch_status();
}

// `scratch` holds R * n_chunks candidates of 8 bytes (n_chunks <= 64), 8-byte aligned.
extern "C" int cvb_sample_chunked(int* out, const float* logits, const int* rows, const float* temps,
                                  const uint64_t* seeds, const int* out_positions, int R, int V, int n_logit_rows,
                                  int n_chunks, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    if (R == 0) return CVB_OK;
    if (R < 0 || V <= 0 || n_logit_rows <= 0 || n_chunks < 1 || n_chunks > 64) return CVB_E_SIZE;
    if (scratch == nullptr || scratch_bytes < static_cast<int64_t>(R) * n_chunks * 8) return CVB_E_SCRATCH;
    if (reinterpret_cast<uintptr_t>(scratch) & 7) return CVB_E_ALIGN;
    unsigned long long* part = static_cast<unsigned long long*>(scratch);
    dim3 grid(static_cast<unsigned>(R), static_cast<unsigned>(n_chunks));
    launch_kernel(sample_search_kernel, dim3(grid), dim3(n_chunks == 1 ? 1024 : 256), 0, stream, out, part, logits, rows, temps, seeds,
                  out_positions, V, n_logit_rows, n_chunks);
    if (n_chunks > 1) launch_kernel(sample_pick_kernel, dim3(R), dim3(32), 0, stream, out, part, V, n_chunks);
    return launch_status();
}

extern "C" int cvb_feed_tokens(int* tokens, const int* src, const int* sampled, int n, int n_sampled,
                               cudaStream_t stream) {
    if (n == 0) return CVB_OK;
    if (n < 0) return CVB_E_SIZE;
    launch_kernel(feed_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, tokens, src, sampled, n, n_sampled);
    return launch_status();
}
