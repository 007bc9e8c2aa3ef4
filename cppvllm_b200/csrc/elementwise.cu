// Embedding gather, RMSNorm, residual-add + RMSNorm, residual add, SwiGLU and row gather.
// General kernels: any row length, float or bf16 activations, float norm weights.
//
// Formulas (reference kernels/fused_ops.cu):
//   rms_norm      :61-88   out = T( rnd(x * rsqrt(mean(x^2) + eps)) * w )
//   add_rms_norm  :70-87   resid = T(resid + x) first, then the norm of the new residual
//   swiglu        :210-220 out = T( rnd(g / (1 + exp(-g))) * u ),  g = gu[r, i], u = gu[r, I + i]
// Sums of squares, rsqrt, the residual sum and the activation are float in both paths.
#include "common.cuh"

namespace cvb {

// One row from `src` to `dst` by the block's threads: 16 bytes at a time where the row's length and both addresses
// allow it (a thread then has several copies in flight), element by element otherwise.
template <typename T>
__device__ __forceinline__ void copy_row(T* __restrict__ dst, const T* __restrict__ src, int D) {
    constexpr int N = 16 / sizeof(T);
    if (D % N == 0 && ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < D / N; i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
    }
}

template <typename T>
__global__ void embed_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ tokens,
                             int D, int V, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= V) {           // never read outside the table: record and clamp
        if (threadIdx.x == 0) atomicExch(err, 1);
        tok = tok < 0 ? 0 : V - 1;
    }
    copy_row(out + t * D, table + static_cast<int64_t>(tok) * D, D);
}

// Rows of any length and alignment (the forms further down need 16-byte rows): a warp owns a row and its lanes walk
// the row's elements; with `add`, the residual stream is updated in place on the first walk and read back on the second.
constexpr int kRowWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
rmsnorm_rows_kernel(T* __restrict__ out, T* stream_io, const T* __restrict__ x, const float* __restrict__ w, int n_rows, int D,
                    float eps, int add) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const T* src = x + row * D;
    T* sum_row = add ? stream_io + row * D : nullptr;
    float sq = 0.f;
    for (int i = lane; i < D; i += 32) {
        float v = to_float(src[i]);
        if (add) {
            v = rnd<T>(to_float(sum_row[i]) + v);
            sum_row[i] = from_float<T>(v);
        }
        sq = fmaf(v, v, sq);
    }
    const float scale = rsqrtf(warp_sum(sq) / static_cast<float>(D) + eps);
    const T* normed_from = add ? sum_row : src;             // lanes read back only what they wrote themselves
    for (int i = lane; i < D; i += 32) out[row * D + i] = from_float<T>(rnd<T>(to_float(normed_from[i]) * scale) * w[i]);
}

template <typename T>
__global__ void add_kernel(T* __restrict__ resid, const T* __restrict__ x, int64_t n) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) resid[i] = from_float<T>(to_float(resid[i]) + to_float(x[i]));
}

template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ in, const int* __restrict__ rows,
                                   int D, int n_in) {
    pdl_trigger();
    pdl_wait();
    const int64_t r = blockIdx.x;
    int src = rows[r];
    if (src < 0) src = 0;
    if (src >= n_in) src = n_in - 1;
    copy_row(out + r * D, in + static_cast<int64_t>(src) * D, D);
}


// ---- 16-byte vector forms (rows whose length is a multiple of the vector width and whose base is aligned) --------

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const {
        uint4 t;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = t;
    }
};

constexpr int kNormThreads = 128;
constexpr int kNormMaxChunks = 8;      // per thread: rows up to 128 * 8 * (4 or 8) elements stay in registers

// Same arithmetic as rmsnorm_rows_kernel, one global read of the row: the (summed) row is kept in registers.
template <typename T, bool ADD>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_vec_kernel(T* __restrict__ out, T* resid, const T* __restrict__ x, const float* __restrict__ w, int D, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    constexpr int N = Vec16<T>::N;
    const int64_t row = blockIdx.x;
    const int n_chunks = D / N;
    Vec16<T> val[kNormMaxChunks];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kNormMaxChunks; ++k) {
        const int c = threadIdx.x + k * kNormThreads;
        if (c < n_chunks) {
            val[k].load(x + row * D + c * N);
            if constexpr (ADD) {
                Vec16<T> r;
                r.load(resid + row * D + c * N);
#pragma unroll
                for (int i = 0; i < N; ++i) val[k].v[i] = rnd<T>(r.v[i] + val[k].v[i]);
                val[k].store(resid + row * D + c * N);
            }
#pragma unroll
            for (int i = 0; i < N; ++i) ss += val[k].v[i] * val[k].v[i];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (int k = 0; k < kNormMaxChunks; ++k) {
        const int c = threadIdx.x + k * kNormThreads;
        if (c < n_chunks) {
            Vec16<T> o;
#pragma unroll
            for (int i = 0; i < N; ++i) o.v[i] = rnd<T>(val[k].v[i] * inv) * w[c * N + i];
            o.store(out + row * D + c * N);
        }
    }
}

// One warp per row, for rows of up to 32 * kWarpNormChunks chunks: several 16-byte loads in flight per lane, the sum
// over the row by shuffles alone.  Same arithmetic as above.
constexpr int kWarpNormChunks = 16;
constexpr int kWarpNormWarps = 4;

template <typename T, bool ADD, int CHUNKS>
__global__ void __launch_bounds__(kWarpNormWarps * 32)
rmsnorm_warp_kernel(T* __restrict__ out, T* resid, const T* __restrict__ x, const float* __restrict__ w, int T_rows, int D, float eps) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpNormWarps + (threadIdx.x >> 5);
    if (row >= T_rows) return;
    const int n_chunks = D / N;
    Vec16<T> val[CHUNKS];
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        const int c = lane + k * 32;
        if (c < n_chunks) val[k].load(x + row * D + c * N);
    }
    if constexpr (ADD) {
        Vec16<T> r[CHUNKS];
#pragma unroll
        for (int k = 0; k < CHUNKS; ++k) {
            const int c = lane + k * 32;
            if (c < n_chunks) r[k].load(resid + row * D + c * N);
        }
#pragma unroll
        for (int k = 0; k < CHUNKS; ++k) {
            const int c = lane + k * 32;
            if (c < n_chunks) {
#pragma unroll
                for (int i = 0; i < N; ++i) val[k].v[i] = rnd<T>(r[k].v[i] + val[k].v[i]);
                val[k].store(resid + row * D + c * N);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        const int c = lane + k * 32;
        if (c < n_chunks) {
#pragma unroll
            for (int i = 0; i < N; ++i) ss += val[k].v[i] * val[k].v[i];
        }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        const int c = lane + k * 32;
        if (c < n_chunks) {
            Vec16<T> o;
#pragma unroll
            for (int i = 0; i < N; i += 4) {
                const float4 ww = *reinterpret_cast<const float4*>(w + c * N + i);
                o.v[i] = rnd<T>(val[k].v[i] * inv) * ww.x;
                o.v[i + 1] = rnd<T>(val[k].v[i + 1] * inv) * ww.y;
                o.v[i + 2] = rnd<T>(val[k].v[i + 2] * inv) * ww.z;
                o.v[i + 3] = rnd<T>(val[k].v[i + 3] * inv) * ww.w;
            }
            o.store(out + row * D + c * N);
        }
    }
}

// launches the warp form with the smallest chunk count that holds the row; false if the row is too long for it
template <typename T, bool ADD>
__host__ bool launch_warp_norm(T* out, T* resid, const T* x, const float* w, int T_rows, int D, float eps, cudaStream_t stream) {
    const int per_lane = (D / Vec16<T>::N + 31) / 32;
    if (per_lane > kWarpNormChunks || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return false;
    // A few long rows (a decode step of a wide model) are a chain of latencies for one warp per row (23 us for one row of
    // 4,096 elements): the form with a block per row spreads a row over 128 threads.
    if (per_lane > 4 && T_rows < 256 && D <= kNormThreads * kNormMaxChunks * Vec16<T>::N) return false;
    const dim3 grid((T_rows + kWarpNormWarps - 1) / kWarpNormWarps), block(kWarpNormWarps * 32);
    if (per_lane <= 1) launch_kernel(rmsnorm_warp_kernel<T, ADD, 1>, grid, block, 0, stream, out, resid, x, w, T_rows, D, eps);
    else if (per_lane <= 2) launch_kernel(rmsnorm_warp_kernel<T, ADD, 2>, grid, block, 0, stream, out, resid, x, w, T_rows, D, eps);
    else if (per_lane <= 4) launch_kernel(rmsnorm_warp_kernel<T, ADD, 4>, grid, block, 0, stream, out, resid, x, w, T_rows, D, eps);
    else if (per_lane <= 8) launch_kernel(rmsnorm_warp_kernel<T, ADD, 8>, grid, block, 0, stream, out, resid, x, w, T_rows, D, eps);
    else launch_kernel(rmsnorm_warp_kernel<T, ADD, 16>, grid, block, 0, stream, out, resid, x, w, T_rows, D, eps);
    return true;
}

// g / (1 + exp(-g)).  In bfloat16 the quotient is rounded to 8 bits of mantissa right away, so the fast exponential and
// division (errors of a few units in the last place of a float) serve; in float32 the exact ones are used.
template <typename T> __device__ __forceinline__ float silu_of(float g) { return g / (1.f + expf(-g)); }
template <> __device__ __forceinline__ float silu_of<__nv_bfloat16>(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// any width: blockIdx.y walks the rows, the block's threads a row's columns
template <typename T>
__global__ void swiglu_rows_kernel(T* __restrict__ out, const T* __restrict__ gu, int n_rows, int I) {
    pdl_trigger();
    pdl_wait();
    for (int64_t row = blockIdx.y; row < n_rows; row += gridDim.y) {
        const T* gate = gu + row * 2 * I;
        T* dst = out + row * I;
        for (int col = blockIdx.x * blockDim.x + threadIdx.x; col < I; col += gridDim.x * blockDim.x)
            dst[col] = from_float<T>(rnd<T>(silu_of<T>(to_float(gate[col]))) * to_float(gate[I + col]));
    }
}

template <typename T>
__global__ void swiglu_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n_chunks, int I) {
    pdl_trigger();
    pdl_wait();
    constexpr int N = Vec16<T>::N;
    const int64_t k = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (k >= n_chunks) return;
    const int per_row = I / N;
    const int64_t r = k / per_row;
    const int i0 = static_cast<int>(k - r * per_row) * N;
    Vec16<T> g, u, o;
    g.load(gu + r * 2 * I + i0);
    u.load(gu + r * 2 * I + I + i0);
#pragma unroll
    for (int i = 0; i < N; ++i) o.v[i] = rnd<T>(silu_of<T>(g.v[i])) * u.v[i];
    o.store(out + r * I + i0);
}

template <typename T> __host__ inline bool vec_ok(const void* a, const void* b, const void* c, int width) {
    constexpr int N = Vec16<T>::N;
    auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return width % N == 0 && al(a) && al(b) && al(c);
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_embed(void* out, const void* table, const int* tokens, int T, int D, int V, int dtype,
                         int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || V <= 0) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(embed_kernel<TY>, dim3(T), dim3(128), 0, stream, (TY*)out, (const TY*)table, tokens, D, V, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_rmsnorm(void* out, const void* x, const float* w, int T, int D, float eps, int dtype,
                           cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0) return CVB_E_SIZE;
#define CALL(TY)                                                                                              \
    if (vec_ok<TY>(out, x, nullptr, D) && launch_warp_norm<TY, false>((TY*)out, nullptr, (const TY*)x, w, T, D, eps, stream)) {} \
    else if (vec_ok<TY>(out, x, nullptr, D) && D <= kNormThreads * kNormMaxChunks * Vec16<TY>::N)             \
        launch_kernel(rmsnorm_vec_kernel<TY, false>, dim3(T), dim3(kNormThreads), 0, stream, (TY*)out, nullptr, (const TY*)x, w, D, eps); \
    else                                                                                                      \
        launch_kernel(rmsnorm_rows_kernel<TY>, dim3((T + kRowWarps - 1) / kRowWarps), dim3(kRowWarps * 32), 0, stream, (TY*)out, nullptr, (const TY*)x, w, T, D, eps, 0)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_add_rmsnorm(void* out, void* resid, const void* x, const float* w, int T, int D, float eps,
                               int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0) return CVB_E_SIZE;
#define CALL(TY)                                                                                              \
    if (vec_ok<TY>(out, x, resid, D) && launch_warp_norm<TY, true>((TY*)out, (TY*)resid, (const TY*)x, w, T, D, eps, stream)) {} \
    else if (vec_ok<TY>(out, x, resid, D) && D <= kNormThreads * kNormMaxChunks * Vec16<TY>::N)               \
        launch_kernel(rmsnorm_vec_kernel<TY, true>, dim3(T), dim3(kNormThreads), 0, stream, (TY*)out, (TY*)resid, (const TY*)x, w, D, eps); \
    else                                                                                                      \
        launch_kernel(rmsnorm_rows_kernel<TY>, dim3((T + kRowWarps - 1) / kRowWarps), dim3(kRowWarps * 32), 0, stream, (TY*)out, (TY*)resid, (const TY*)x, w, T, D, eps, 1)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_add(void* resid, const void* x, int64_t n, int dtype, cudaStream_t stream) {
    if (n == 0) return CVB_OK;
    if (n < 0) return CVB_E_SIZE;
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
#define CALL(TY) launch_kernel(add_kernel<TY>, dim3(blocks), dim3(256), 0, stream, (TY*)resid, (const TY*)x, n)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_swiglu(void* out, const void* gate_up, int T, int I, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || I <= 0) return CVB_E_SIZE;
    const int64_t n = static_cast<int64_t>(T) * I;
#define CALL(TY)                                                                                              \
    if (vec_ok<TY>(out, gate_up, nullptr, I)) {                                                               \
        const int64_t nc = n / Vec16<TY>::N;                                                                  \
        launch_kernel(swiglu_vec_kernel<TY>, dim3(static_cast<unsigned>((nc + 255) / 256)), dim3(256), 0, stream, (TY*)out, (const TY*)gate_up, nc, I); \
    } else                                                                                                    \
        launch_kernel(swiglu_rows_kernel<TY>, dim3(static_cast<unsigned>(min(64, (I + 255) / 256)), static_cast<unsigned>(min(T, 65535))), dim3(256), 0, stream, (TY*)out, (const TY*)gate_up, T, I)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_gather_rows(void* out, const void* in, const int* rows, int R, int D, int n_in, int dtype,
                               cudaStream_t stream) {
    if (R == 0) return CVB_OK;
    if (R < 0 || D <= 0 || n_in <= 0) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(gather_rows_kernel<TY>, dim3(R), dim3(128), 0, stream, (TY*)out, (const TY*)in, rows, D, n_in)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
