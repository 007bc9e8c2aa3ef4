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
    using Raw = float4;
    static __device__ __forceinline__ Raw load_raw(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void unpack(float (&v)[4], const Raw& t) { v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    static __device__ __forceinline__ void round_all(float (&)[4]) {}
    static __device__ __forceinline__ void load(float (&v)[4], const float* p) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
    static __device__ __forceinline__ void store_raw(float* p, const Raw& t) { *reinterpret_cast<float4*>(p) = t; }
    // the partner lane's values (lane ^ delta)
    static __device__ __forceinline__ void exchange(float (&other)[4], const float (&v)[4], int delta) {
#pragma unroll
        for (int i = 0; i < 4; ++i) other[i] = __shfl_xor_sync(0xffffffffu, v[i], delta);
    }
};
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int N = 8;
    using Raw = uint4;
    static __device__ __forceinline__ Raw load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
    // round every element to bf16 and back, two at a time (one packed conversion and two bit operations per pair)
    static __device__ __forceinline__ void round_all(float (&v)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[i], v[i + 1]);
            const uint32_t bits = *reinterpret_cast<const uint32_t*>(&h);
            v[i] = __uint_as_float(bits << 16);
            v[i + 1] = __uint_as_float(bits & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void unpack(float (&v)[8], const Raw& t) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
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
    static __device__ __forceinline__ void store_raw(__nv_bfloat16* p, const Raw& t) { *reinterpret_cast<uint4*>(p) = t; }
    // the partner lane's values (lane ^ delta); the values are exact in bf16 here, so they travel two to a word
    static __device__ __forceinline__ void exchange(float (&other)[8], const float (&v)[8], int delta) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const uint32_t mine = (__float_as_uint(v[i]) >> 16) | (__float_as_uint(v[i + 1]) & 0xffff0000u);
            const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, delta);
            other[i] = __uint_as_float(theirs << 16);
            other[i + 1] = __uint_as_float(theirs & 0xffff0000u);
        }
    }
};

constexpr int kVecThreads = 128;

// One block per token: its threads walk the token's heads (q heads, then k, then v) kVecThreads / CH at a time, so
// the token's position, slot, rotation angles and norm weights are fetched once, and the loads of several heads are in
// flight together.
template <typename T, int CH>
__global__ void __launch_bounds__(kVecThreads)
qk_norm_rope_kv_vec_kernel(T* __restrict__ q_out, const T* __restrict__ qkv, const float* __restrict__ q_w,
                           const float* __restrict__ k_w, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                           const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ cache,
                           int H, int KV, int page_size, int max_pos, float eps, int64_t cache_elems,
                           int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = Chunk<T>::N;
    constexpr int hd = CH * N;
    constexpr int per_round = kVecThreads / CH;
    const int sub = threadIdx.x / CH, c = threadIdx.x % CH;
    const int n_tasks = H + 2 * KV;
    const int64_t t = blockIdx.x;
    const int slot = slots ? slots[t] : -1;
    const bool first = c < (CH >> 1);
    const int rounds = (n_tasks + per_round - 1) / per_round;
    // the head vectors of the first rounds are requested before anything that depends on the token's position or
    // slot, so that the two latencies overlap
    constexpr int kBatch = 4;
    const T* src_row = qkv + t * n_tasks * hd + c * N;
    typename Chunk<T>::Raw raw[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) raw[k] = Chunk<T>::load_raw(src_row + min(k * per_round + sub, n_tasks - 1) * hd);
    float cs[N], sn[N], wq[N], wk[N];
#pragma unroll
    for (int i = 0; i < N; ++i) { cs[i] = 1.f; sn[i] = 0.f; wq[i] = 1.f; wk[i] = 1.f; }
    if (cos_t != nullptr) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) {
            if (threadIdx.x == 0) atomicExch(err, 3);
            pos = pos < 0 ? 0 : max_pos - 1;
        }
        const int e0 = (first ? c : c - (CH >> 1)) * N;
        const float* cr = cos_t + static_cast<int64_t>(pos) * (hd >> 1) + e0;
        const float* sr = sin_t + static_cast<int64_t>(pos) * (hd >> 1) + e0;
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            const float4 a = *reinterpret_cast<const float4*>(cr + i), b = *reinterpret_cast<const float4*>(sr + i);
            cs[i] = a.x; cs[i + 1] = a.y; cs[i + 2] = a.z; cs[i + 3] = a.w;
            sn[i] = b.x; sn[i + 1] = b.y; sn[i + 2] = b.z; sn[i + 3] = b.w;
        }
        if (first) {                                              // first half: x cos - other sin; second: x cos + other sin
#pragma unroll
            for (int i = 0; i < N; ++i) sn[i] = -sn[i];
        }
    }
    if (q_w != nullptr) {
#pragma unroll
        for (int i = 0; i < N; ++i) { wq[i] = q_w[c * N + i]; wk[i] = k_w[c * N + i]; }
    }
    // what does not change from head to head is computed once: the row of this token in q_out, and the row of its slot
    // in the K block of its page (the V block lies KV * page_size rows further, head kvh page_size rows further)
    T* q_row = q_out + t * H * hd + c * N;
    int64_t k_row = -1;
    if (slot >= 0 && cache != nullptr) {
        const int page = slot / page_size, off = slot - page * page_size;
        k_row = static_cast<int64_t>(page) * 2 * KV * page_size + off;
        if ((k_row + (2 * KV - 1) * static_cast<int64_t>(page_size) + 1) * hd > cache_elems) {
            if (threadIdx.x == 0) atomicExch(err, 2);
            k_row = -1;
        }
    }
    const float inv_hd = 1.f / static_cast<float>(hd);
    for (int round0 = 0; round0 < rounds; round0 += kBatch) {
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const int round = round0 + k;
            if (round >= rounds) break;                           // uniform over the block
            const int task_raw = round * per_round + sub;
            const bool active = task_raw < n_tasks;
            const int task = active ? task_raw : n_tasks - 1;       // idle lanes hold a valid vector and store nothing
            const bool is_q = task < H, is_v = task >= H + KV;
            if (round * per_round >= H + KV) {
                // the whole round holds value heads (uniform over the block): they are copied as they are
                if (active && k_row >= 0)
                    Chunk<T>::store_raw(cache + (k_row + static_cast<int64_t>(task - H) * page_size) * hd + c * N, raw[k]);
                if (round + kBatch < rounds)
                    raw[k] = Chunk<T>::load_raw(src_row + min((round + kBatch) * per_round + sub, n_tasks - 1) * hd);
                continue;
            }
            float x[N];
            Chunk<T>::unpack(x, raw[k]);
            if (round + kBatch < rounds)                          // the same slot of the next batch
                raw[k] = Chunk<T>::load_raw(src_row + min((round + kBatch) * per_round + sub, n_tasks - 1) * hd);
            T* dst = nullptr;                                     // destination of this chunk (nullptr: nothing to write)
            if (active) {
                if (is_q) dst = q_row + task * hd;
                else if (k_row >= 0) dst = cache + (k_row + static_cast<int64_t>(task - H) * page_size) * hd + c * N;
            }
            if (is_v) {
                if (dst != nullptr) Chunk<T>::store(dst, x);
#pragma unroll
                for (int i = 0; i < N; ++i) x[i] = 0.f;
            }
            // all lanes take part in the shuffles below
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < N; ++i) ss += x[i] * x[i];
#pragma unroll
            for (int o = CH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (q_w != nullptr) {
                const float inv = rsqrtf(ss * inv_hd + eps);
#pragma unroll
                for (int i = 0; i < N; ++i) x[i] *= inv;
                Chunk<T>::round_all(x);
#pragma unroll
                for (int i = 0; i < N; ++i) x[i] *= is_q ? wq[i] : wk[i];
                Chunk<T>::round_all(x);
            }
            float other[N];
            if (q_w != nullptr) {
                Chunk<T>::exchange(other, x, CH >> 1);            // normed values are exact in the activation type
            } else {
#pragma unroll
                for (int i = 0; i < N; ++i) other[i] = __shfl_xor_sync(0xffffffffu, x[i], CH >> 1);
            }
            if (is_v || dst == nullptr) continue;
            if (cos_t != nullptr) {
                float out[N];
#pragma unroll
                for (int i = 0; i < N; ++i) out[i] = x[i] * cs[i] + other[i] * sn[i];
                Chunk<T>::store(dst, out);
            } else {
                Chunk<T>::store(dst, x);
            }
        }
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
            dim3 vgrid(static_cast<unsigned>(T));
#define VCALL_CH(TY, C)                                                                                        \
    launch_kernel(qk_norm_rope_kv_vec_kernel<TY, C>, dim3(vgrid), dim3(kVecThreads), 0, stream,                                      \
        (TY*)q_out, (const TY*)qkv, q_w, k_w, cos_t, sin_t, positions, slots, (TY*)cache, H, KV,              \
        page_size, max_pos, eps, cache_elems, err_flag)
#define VCALL(TY)                                                                                             \
    switch (CH) {                                                                                             \
        case 2: VCALL_CH(TY, 2); break;                                                                       \
        case 4: VCALL_CH(TY, 4); break;                                                                       \
        case 8: VCALL_CH(TY, 8); break;                                                                       \
        case 16: VCALL_CH(TY, 16); break;                                                                     \
        default: VCALL_CH(TY, 32); break;                                                                     \
    }
            CVB_DISPATCH_DTYPE(dtype, VCALL);
#undef VCALL
#undef VCALL_CH
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
