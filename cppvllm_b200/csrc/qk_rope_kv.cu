// Fused per-head RMSNorm of q and k, rotary position encoding, and the write of k and v into cache pages.
//
// One warp owns one (token, head) vector of the packed projection row [q: H*hd | k: KV*hd | v: KV*hd].
// Formulas (reference kernels/fused_ops.cu:104-207, without its FP8 quantisation):
//   q, k :  n = rnd( rnd(x * rsqrt(mean_hd(x^2) + eps)) * w )         one weight vector for all heads
//           rotate-half pairs (i, i + rot/2):  out_i = n_i cos - n_{i+rot/2} sin,  out_{i+rot/2} = n_{i+rot/2} cos + n_i sin
//           with cos/sin read from float tables [max_pos, rot/2] at the token's absolute position
//   v    :  copied unchanged
//   k, v land at cache[page, 0|1, kv_head, slot % page_size, :] with page = slot / page_size; a negative slot
//   skips the write (a layer that reads another layer's cache computes q only).
// General in head size (any even hd), rotary width (rot <= hd, even), pairing (rotate-half or interleaved),
// with or without the per-head norm and with or without rotation.
#include "common.cuh"

namespace cvb {

constexpr int kWarpsPerBlock = 4;

template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ q_out, const T* __restrict__ qkv,
                                       const float* __restrict__ q_w, const float* __restrict__ k_w,
                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       T* __restrict__ cache, int H, int KV, int hd, int rot, int interleaved,
                                       int page_size, int max_pos, float eps, int64_t cache_elems,
                                       int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int task = blockIdx.y * kWarpsPerBlock + warp;
    const int n_tasks = H + 2 * KV;
    if (task >= n_tasks) return;
    float* buf = smem + warp * hd;
    const int64_t t = blockIdx.x;
    const T* src = qkv + (t * n_tasks + task) * hd;
    const int slot = slots ? slots[t] : -1;

    if (task >= H + KV) {                                  // v: copy into its page
        if (slot < 0 || cache == nullptr) return;
        const int kvh = task - H - KV;
        const int64_t page = slot / page_size, off = slot % page_size;
        const int64_t base = (((page * 2 + 1) * KV + kvh) * page_size + off) * hd;
        if (base + hd > cache_elems) { if (lane == 0) atomicExch(err, 2); return; }
        for (int e = lane; e < hd; e += 32) cache[base + e] = src[e];
        return;
    }

    const bool is_q = task < H;
    if (!is_q && (slot < 0 || cache == nullptr)) return;   // k of a layer that does not write its cache
    const float* w = is_q ? q_w : k_w;

    float ss = 0.f;
    for (int e = lane; e < hd; e += 32) { const float x = to_float(src[e]); buf[e] = x; ss += x * x; }
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / static_cast<float>(hd) + eps);
        for (int e = lane; e < hd; e += 32) buf[e] = rnd<T>(rnd<T>(buf[e] * inv) * w[e]);
    }
    __syncwarp();

    T* dst;
    if (is_q) {
        dst = q_out + (t * H + task) * hd;
    } else {
        const int kvh = task - H;
        const int64_t page = slot / page_size, off = slot % page_size;
        const int64_t base = (((page * 2 + 0) * KV + kvh) * page_size + off) * hd;
        if (base + hd > cache_elems) { if (lane == 0) atomicExch(err, 2); return; }
        dst = cache + base;
    }

    const int half = rot >> 1;
    if (cos_t != nullptr && half > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) {                   // outside the tables: record and clamp
            if (lane == 0) atomicExch(err, 3);
            pos = pos < 0 ? 0 : max_pos - 1;
        }
        const float* c_row = cos_t + static_cast<int64_t>(pos) * half;
        const float* s_row = sin_t + static_cast<int64_t>(pos) * half;
        for (int i = lane; i < half; i += 32) {
            const int ia = interleaved ? 2 * i : i;
            const int ib = interleaved ? 2 * i + 1 : i + half;
            const float c = c_row[i], s = s_row[i];
            const float a = buf[ia], b = buf[ib];
            dst[ia] = from_float<T>(a * c - b * s);
            dst[ib] = from_float<T>(b * c + a * s);
        }
        for (int e = rot + lane; e < hd; e += 32) dst[e] = from_float<T>(buf[e]);
    } else {
        for (int e = lane; e < hd; e += 32) dst[e] = from_float<T>(buf[e]);
    }
}


// ---- 16-byte vector form: head sizes whose chunk count is a power of two, full-width rotate-half rotation --------
//
// One thread owns one 16-byte chunk of a head vector; the hd / N threads of a head are neighbours in a warp, so the
// sum of squares is a butterfly over the group and the rotation partner (element i + hd/2) lives in lane ^ (CH/2).
template <typename T> struct Chunk;
template <> struct Chunk<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(float (&v)[4], const float* p) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(float (&v)[8], const __nv_bfloat16* p) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 t;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = t;
    }
};

constexpr int kVecThreads = 128;

template <typename T>
__global__ void __launch_bounds__(kVecThreads)
qk_norm_rope_kv_vec_kernel(T* __restrict__ q_out, const T* __restrict__ qkv, const float* __restrict__ q_w,
                           const float* __restrict__ k_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                           const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ cache,
                           int H, int KV, int hd, int CH, int page_size, int max_pos, float eps, int64_t cache_elems,
                           int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = Chunk<T>::N;
    const int tasks_per_block = kVecThreads / CH;
    const int task = blockIdx.y * tasks_per_block + threadIdx.x / CH;
    const int c = threadIdx.x % CH;
    const int n_tasks = H + 2 * KV;
    const int64_t t = blockIdx.x;
    const bool active = task < n_tasks;
    const int slot = slots ? slots[t] : -1;
    const bool is_q = task < H, is_v = task >= H + KV;
    float x[N];
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = 0.f;
    if (active) Chunk<T>::load(x, qkv + (t * n_tasks + task) * hd + c * N);

    // destination of this chunk (nullptr: nothing to write)
    T* dst = nullptr;
    if (active) {
        if (is_q) {
            dst = q_out + (t * H + task) * hd + c * N;
        } else if (slot >= 0 && cache != nullptr) {
            const int kvh = is_v ? task - H - KV : task - H;
            const int64_t page = slot / page_size, off = slot % page_size;
            const int64_t base = (((page * 2 + (is_v ? 1 : 0)) * KV + kvh) * page_size + off) * hd;
            if (base + hd > cache_elems) { if (c == 0) atomicExch(err, 2); }
            else dst = cache + base + c * N;
        }
    }
    if (active && is_v) {
        if (dst != nullptr) Chunk<T>::store(dst, x);
    }
    // all lanes take part in the shuffles below; v tasks and idle lanes carry zeros
    const float* w = is_q ? q_w : k_w;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) ss += x[i] * x[i];
    for (int o = CH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (w != nullptr && active && !is_v) {
        const float inv = rsqrtf(ss / static_cast<float>(hd) + eps);
#pragma unroll
        for (int i = 0; i < N; ++i) x[i] = rnd<T>(rnd<T>(x[i] * inv) * w[c * N + i]);
    }
    float other[N];
#pragma unroll
    for (int i = 0; i < N; ++i) other[i] = __shfl_xor_sync(0xffffffffu, x[i], CH >> 1);
    if (!active || is_v || dst == nullptr) return;
    if (cos_t != nullptr) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) {
            if (c == 0) atomicExch(err, 3);
            pos = pos < 0 ? 0 : max_pos - 1;
        }
        const bool first = c < (CH >> 1);
        const int e0 = (first ? c : c - (CH >> 1)) * N;
        const float* cr = cos_t + static_cast<int64_t>(pos) * (hd >> 1) + e0;
        const float* sr = sin_t + static_cast<int64_t>(pos) * (hd >> 1) + e0;
        float out[N];
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float cs = cr[i], sn = sr[i];
            out[i] = first ? x[i] * cs - other[i] * sn : x[i] * cs + other[i] * sn;
        }
        Chunk<T>::store(dst, out);
    } else {
        Chunk<T>::store(dst, x);
    }
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_qk_norm_rope_kv(void* q_out, const void* qkv, const float* q_w, const float* k_w,
                                   const float* cos_t, const float* sin_t, const int* positions, const int* slots,
                                   void* cache, int T, int H, int KV, int hd, int rot, int interleaved,
                                   int page_size, int max_pos, float eps, int64_t cache_elems, int dtype,
                                   int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || KV <= 0 || hd <= 0 || page_size <= 0) return CVB_E_SIZE;
    if (hd > 1024) return CVB_E_SIZE;
    if (rot < 0 || rot > hd || (rot & 1)) return CVB_E_SHAPE;
    if ((q_w == nullptr) != (k_w == nullptr)) return CVB_E_SHAPE;
    if (cos_t != nullptr && (sin_t == nullptr || positions == nullptr || max_pos <= 0)) return CVB_E_SHAPE;
    const int n_tasks = H + 2 * KV;
    {   // vector form when the head splits into a power-of-two number (2..32) of aligned 16-byte chunks
        const int esize = dtype == CVB_DTYPE_BF16 ? 2 : 4;
        const int N = 16 / esize;
        const int CH = hd % N == 0 ? hd / N : 0;
        auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
        const bool full_rot = cos_t == nullptr || (rot == hd && !interleaved);
        if (CH >= 2 && CH <= 32 && (CH & (CH - 1)) == 0 && full_rot && al(q_out) && al(qkv) && al(cache) && al(cos_t) &&
            al(sin_t) && (dtype == CVB_DTYPE_BF16 || dtype == CVB_DTYPE_F32)) {
            const int tasks_per_block = kVecThreads / CH;
            dim3 vgrid(static_cast<unsigned>(T), static_cast<unsigned>((n_tasks + tasks_per_block - 1) / tasks_per_block));
#define VCALL(TY)                                                                                             \
    launch_kernel(qk_norm_rope_kv_vec_kernel<TY>, dim3(vgrid), dim3(kVecThreads), 0, stream,                                         \
        (TY*)q_out, (const TY*)qkv, q_w, k_w, cos_t, sin_t, positions, slots, (TY*)cache, H, KV, hd, CH,       \
        page_size, max_pos, eps, cache_elems, err_flag)
            CVB_DISPATCH_DTYPE(dtype, VCALL);
#undef VCALL
            return launch_status();
        }
    }
    dim3 grid(static_cast<unsigned>(T), static_cast<unsigned>((n_tasks + kWarpsPerBlock - 1) / kWarpsPerBlock));
    const size_t smem = static_cast<size_t>(kWarpsPerBlock) * hd * sizeof(float);
#define CALL(TY)                                                                                              \
    launch_kernel(qk_norm_rope_kv_kernel<TY>, dim3(grid), dim3(kWarpsPerBlock * 32), smem, stream,                                   \
        (TY*)q_out, (const TY*)qkv, q_w, k_w, cos_t, sin_t, positions, slots, (TY*)cache, H, KV, hd, rot,      \
        interleaved, page_size, max_pos, eps, cache_elems, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
