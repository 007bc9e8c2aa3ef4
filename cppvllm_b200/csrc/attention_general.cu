// General paged attention: any head size, any number of heads and groups, float or bf16, optional window.
// One block per (query token, query head).  It serves prompt portions and decoded tokens alike, because
// every query token is handled on its own: its keys are those of its request at positions lo..p, read
// through the request's block table, where p is the token's absolute position and lo = 0 or, with a
// window w > 0, max(0, p - w + 1).  The keys of the step's own tokens are already in the pages (the
// projection kernel writes before this kernel reads).
//
// Formulas (reference kernels/paged_attention.cu:89-359 and model/model_architecture.cpp:134,147):
//   query head h uses kv head h / (H / KV);  s_j = scale * q . k_j  for lo <= j <= p, others excluded;
//   running maximum m, sum l and accumulator in float with expf;  o = sum_j p_j v_j / l;  rounded to T.
// Keys are walked in tiles of blockDim.x from lo, so the order of the float sums depends only on (lo, p):
// not on how the prompt was cut into steps, nor on the batch, nor on which pages hold the keys.
#include "common.cuh"

namespace cvb {

constexpr int kAttnThreads = 128;
constexpr int kMaxDimsPerThread = 8;     // head sizes up to 1024

template <typename T>
__global__ void __launch_bounds__(kAttnThreads)
paged_attention_general_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ cache,
                               const int* __restrict__ block_tables, int table_width,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               int H, int KV, int hd, int page_size, int window, float scale, int num_pages,
                               int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int64_t smem64[];
    int64_t* v_off = smem64;                            // [kAttnThreads]
    float* probs = reinterpret_cast<float*>(v_off + kAttnThreads);   // [kAttnThreads]
    float* scratch = probs + kAttnThreads;              // [32]
    float* qs = scratch + 32;                           // [hd]

    const int64_t t = blockIdx.x;
    const int h = blockIdx.y;
    const int kvh = h / (H / KV);
    const int tid = threadIdx.x;
    const int seq = seq_of_token[t];
    const int p = positions[t];
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int* table = block_tables + static_cast<int64_t>(seq) * table_width;

    for (int e = tid; e < hd; e += kAttnThreads) qs[e] = to_float(q[(t * H + h) * hd + e]);
    __syncthreads();

    float acc[kMaxDimsPerThread];
#pragma unroll
    for (int i = 0; i < kMaxDimsPerThread; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int start = lo; start <= p; start += kAttnThreads) {
        const int j = start + tid;
        float s = -INFINITY;
        int64_t voff = -1;
        if (j <= p) {
            const int slot = j / page_size;
            int page = slot < table_width ? table[slot] : -1;
            if (page < 0 || page >= num_pages) {
                atomicExch(err, 4);                     // a key this token must see has no page
            } else {
                const int64_t koff = (((static_cast<int64_t>(page) * 2 + 0) * KV + kvh) * page_size + j % page_size) * hd;
                voff = (((static_cast<int64_t>(page) * 2 + 1) * KV + kvh) * page_size + j % page_size) * hd;
                const T* kp = cache + koff;
                float d = 0.f;
                for (int e = 0; e < hd; ++e) d = fmaf(qs[e], to_float(kp[e]), d);
                s = d * scale;
            }
        }
        const float tile_max = block_max(s, scratch);
        const float m_new = fmaxf(m, tile_max);
        const float pj = (s == -INFINITY || m_new == -INFINITY) ? 0.f : expf(s - m_new);
        probs[tid] = pj;
        v_off[tid] = voff;
        const float tile_sum = block_sum(pj, scratch);  // also orders the writes above before the reads below
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + tile_sum;
        const int n = min(kAttnThreads, p - start + 1);
#pragma unroll
        for (int i = 0; i < kMaxDimsPerThread; ++i) {
            const int d = tid + i * kAttnThreads;
            if (d < hd) {
                float a = acc[i] * corr;
                for (int jj = 0; jj < n; ++jj) {
                    const int64_t vo = v_off[jj];
                    if (vo >= 0) a = fmaf(probs[jj], to_float(cache[vo + d]), a);
                }
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerThread; ++i) {
        const int d = tid + i * kAttnThreads;
        if (d < hd) out[(t * H + h) * hd + d] = from_float<T>(acc[i] * inv_l);
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_paged_attention_general(void* out, const void* q, const void* cache, const int* block_tables,
                                           int table_width, const int* seq_of_token, const int* positions, int T,
                                           int H, int KV, int hd, int page_size, int window, float scale,
                                           int num_pages, int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || KV <= 0 || hd <= 0 || page_size <= 0 || table_width <= 0 || num_pages <= 0)
        return CVB_E_SIZE;
    if (hd > kAttnThreads * kMaxDimsPerThread) return CVB_E_SIZE;
    if (H % KV) return CVB_E_SHAPE;
    if (H > 65535) return CVB_E_SIZE;
    dim3 grid(static_cast<unsigned>(T), static_cast<unsigned>(H));
    const size_t smem = kAttnThreads * sizeof(int64_t) + (static_cast<size_t>(hd) + kAttnThreads + 32) * sizeof(float);
#define CALL(TY)                                                                                         \
    launch_kernel(paged_attention_general_kernel<TY>, dim3(grid), dim3(kAttnThreads), smem, stream,                             \
        (TY*)out, (const TY*)q, (const TY*)cache, block_tables, table_width, seq_of_token, positions, H, \
        KV, hd, page_size, window, scale, num_pages, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
