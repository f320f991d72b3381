// Residual add + RMSNorm in one pass over the hidden state.
//
// The decoder layer of the reference does `h = h + sublayer(...)` followed by Qwen2RMSNorm on the
// result (spikeinfer/modeling_fast.py:206-211); as separate PyTorch operators that is about ten
// launches per norm.  Here one warp owns a row: it adds the optional delta (rounded to the model
// dtype, as the eager add does), writes the new residual back, accumulates the fp32 sum of squares,
// and writes weight * (x * rsqrt(mean + eps)).to(dtype), i.e. Qwen2RMSNorm's arithmetic.
#include "spk_common.cuh"

namespace {

constexpr int kNormWarps = 8;

template <typename T>
__device__ __forceinline__ float norm_round(float v);
template <>
__device__ __forceinline__ float norm_round<float>(float v) { return v; }
template <>
__device__ __forceinline__ float norm_round<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float norm_round<__half>(float v) { return __half2float(__float2half_rn(v)); }

template <typename T>
__device__ __forceinline__ T norm_cast(float v);
template <>
__device__ __forceinline__ float norm_cast<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 norm_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half norm_cast<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kNormWarps * 32)
add_rmsnorm_kernel(T* __restrict__ h, const T* __restrict__ delta, const T* __restrict__ weight, float eps,
                   T* __restrict__ out, int64_t rows, int hidden) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    T* hr = h + row * hidden;
    const T* dr = delta != nullptr ? delta + row * hidden : nullptr;
    T* orow = out + row * hidden;
    float ss = 0.0f;
    for (int c = lane; c < hidden; c += 32) {
        float v = spk_to_float<T>(hr[c]);
        if (dr != nullptr) {
            v = norm_round<T>(__fadd_rn(v, spk_to_float<T>(dr[c])));
            hr[c] = norm_cast<T>(v);
        }
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
    for (int c = lane; c < hidden; c += 32) {
        const float y = norm_round<T>(spk_to_float<T>(hr[c]) * inv);
        orow[c] = norm_cast<T>(spk_to_float<T>(weight[c]) * y);
    }
}

// Fast path: one CTA of 128 threads per row, 16-byte accesses, the row kept in registers between the
// two passes (hidden <= 128 * 8 * kVecPerThread).  Small decode batches have few rows, so a row is
// spread over a whole CTA to keep the dependent-latency chain short.
constexpr int kRowThreads = 128;
constexpr int kVecPerThread = 4;

template <typename T>
struct Vec8 {
    static constexpr int N = 16 / sizeof(T);  // elements per 16-byte access
};

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
add_rmsnorm_row_kernel(T* __restrict__ h, const T* __restrict__ delta, const T* __restrict__ weight, float eps,
                       T* __restrict__ out, int hidden) {
    constexpr int E = Vec8<T>::N;
    __shared__ float part[kRowThreads / 32];
    const int64_t row = blockIdx.x;
    T* hr = h + row * hidden;
    const T* dr = delta != nullptr ? delta + row * hidden : nullptr;
    const int n_vec = hidden / E;
    // the norm weights: in flight together with the row
    uint4 wraw[kVecPerThread];
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
        const int i = threadIdx.x + k * kRowThreads;
        wraw[k] = i < n_vec ? __ldg(reinterpret_cast<const uint4*>(weight + i * E)) : make_uint4(0, 0, 0, 0);
    }
    float v[kVecPerThread][E];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
        const int i = threadIdx.x + k * kRowThreads;
        if (i < n_vec) {
            uint4 raw = *reinterpret_cast<const uint4*>(hr + i * E);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int j = 0; j < E; ++j) v[k][j] = spk_to_float<T>(e[j]);
            if (dr != nullptr) {
                uint4 draw = __ldg(reinterpret_cast<const uint4*>(dr + i * E));
                const T* de = reinterpret_cast<const T*>(&draw);
                T* we = reinterpret_cast<T*>(&raw);
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    v[k][j] = norm_round<T>(__fadd_rn(v[k][j], spk_to_float<T>(de[j])));
                    we[j] = norm_cast<T>(v[k][j]);
                }
                *reinterpret_cast<uint4*>(hr + i * E) = raw;
            }
#pragma unroll
            for (int j = 0; j < E; ++j) ss = fmaf(v[k][j], v[k][j], ss);
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) total += part[w];
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
        const int i = threadIdx.x + k * kRowThreads;
        if (i < n_vec) {
            const T* we = reinterpret_cast<const T*>(&wraw[k]);
            uint4 oraw;
            T* oe = reinterpret_cast<T*>(&oraw);
#pragma unroll
            for (int j = 0; j < E; ++j)
                oe[j] = norm_cast<T>(spk_to_float<T>(we[j]) * norm_round<T>(v[k][j] * inv));
            *reinterpret_cast<uint4*>(out + row * hidden + i * E) = oraw;
        }
    }
}

template <typename T>
int launch_norm(void* h, const void* delta, const void* weight, float eps, void* out, int64_t rows, int hidden,
                cudaStream_t stream) {
    constexpr int E = Vec8<T>::N;
    const bool aligned = reinterpret_cast<uintptr_t>(h) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(weight) % 16 == 0 &&
                         (delta == nullptr || reinterpret_cast<uintptr_t>(delta) % 16 == 0);
    if (aligned && hidden % E == 0 && hidden / E <= kRowThreads * kVecPerThread && rows <= 0x7fffffffLL) {
        add_rmsnorm_row_kernel<T><<<static_cast<unsigned>(rows), kRowThreads, 0, stream>>>(
            static_cast<T*>(h), static_cast<const T*>(delta), static_cast<const T*>(weight), eps,
            static_cast<T*>(out), hidden);
        SPK_CHECK_LAUNCH();
        return SPK_OK;
    }
    const int64_t blocks = (rows + kNormWarps - 1) / kNormWarps;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    add_rmsnorm_kernel<T><<<static_cast<unsigned>(blocks), kNormWarps * 32, 0, stream>>>(
        static_cast<T*>(h), static_cast<const T*>(delta), static_cast<const T*>(weight), eps, static_cast<T*>(out),
        rows, hidden);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace

extern "C" int spk_add_rmsnorm(void* h, const void* delta, const void* weight, float eps, void* out, int64_t rows,
                               int64_t hidden, int dtype, void* stream) {
    SpkRange nvtx_range("spk_add_rmsnorm");
    if (rows < 0 || hidden < 1 || hidden > 0x7fffffffLL) return SPK_ERR_BAD_SHAPE;
    if (rows == 0) return SPK_OK;
    if (h == nullptr || weight == nullptr || out == nullptr) return SPK_ERR_NULL_POINTER;
    cudaStream_t s = spk_stream(stream);
    switch (dtype) {
        case SPK_F32: return launch_norm<float>(h, delta, weight, eps, out, rows, static_cast<int>(hidden), s);
        case SPK_BF16: return launch_norm<__nv_bfloat16>(h, delta, weight, eps, out, rows, static_cast<int>(hidden), s);
        case SPK_F16: return launch_norm<__half>(h, delta, weight, eps, out, rows, static_cast<int>(hidden), s);
        default: return SPK_ERR_BAD_DTYPE;
    }
}
