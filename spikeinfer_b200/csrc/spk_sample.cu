// Greedy sampling inside the captured decode step: argmax over the vocabulary of every row of logits.
//
// The reference samples on the host side of a device sync (spikeinfer/engine/sampler.py:63-81,
// `logits.argmax(dim=-1)` followed by `.tolist()`); here the argmax is two small launches with fixed
// arguments, so it is part of the decode graph.  Semantics of torch.argmax: the first index of the
// largest value, NaN counting as larger than everything.
#include "spk_common.cuh"

namespace {

constexpr int kArgmaxThreads = 256;
constexpr int kArgmaxSplit = 16;  // column ranges per row: rows x 16 CTAs stream the logits

// Candidates are compared as (key, index): the key is an order-preserving integer image of the value in
// which NaN is the largest and -0 equals +0, so "larger key, then smaller index" is torch.argmax's order.
struct Best {
    uint32_t k;
    int64_t i;
};

__device__ __forceinline__ uint32_t order_key(float v) {
    if (v != v) return 0xffffffffu;
    const uint32_t b = __float_as_uint(v + 0.0f);  // -0 -> +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ bool argmax_better(const Best& a, const Best& b) {
    return a.k > b.k || (a.k == b.k && a.i < b.i);
}

__device__ __forceinline__ Best warp_best(Best mine, int width) {
    for (int o = width >> 1; o >= 1; o >>= 1) {
        Best other;
        other.k = __shfl_xor_sync(0xffffffffu, mine.k, o);
        other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
        if (argmax_better(other, mine)) mine = other;
    }
    return mine;
}

template <typename T>
struct Vec;  // 16-byte group of elements
template <>
struct Vec<float> {
    static constexpr int N = 4;
    float4 v;
    __device__ __forceinline__ float get(int i) const { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
};
template <>
struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    uint4 v;
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
};
template <>
struct Vec<__half> {
    static constexpr int N = 8;
    uint4 v;
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
        return __half2float(__ushort_as_half(static_cast<unsigned short>((i & 1) ? (w >> 16) : (w & 0xffffu))));
    }
};

// Pass 1: CTA (range, row) scans its column range; one candidate per CTA.  VEC: rows are 16-byte aligned and
// `per` is a multiple of the group size, so the range is read in 16-byte groups, four per thread in flight.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_partial_kernel(const T* __restrict__ x, int64_t row_stride, int64_t cols, int64_t per,
                      uint32_t* __restrict__ part_k, int64_t* __restrict__ part_i) {
    const int64_t row = blockIdx.y;
    const int64_t lo = per * blockIdx.x;
    const int64_t hi = lo + per < cols ? lo + per : cols;
    const T* xr = x + row * row_stride;
    Best mine{0u, INT64_MAX};
    auto offer = [&](float v, int64_t c) {
        const uint32_t k = order_key(v);
        if (k > mine.k || mine.i == INT64_MAX) { mine.k = k; mine.i = c; }  // ascending c: ties keep the first
    };
    int64_t c = lo;
    if (VEC) {
        constexpr int N = Vec<T>::N;
        const int64_t groups = (hi > lo ? hi - lo : 0) / N;
        const Vec<T>* xv = reinterpret_cast<const Vec<T>*>(xr + lo);
        constexpr int UNROLL = 4;
        int64_t g = threadIdx.x;
        for (; g + (UNROLL - 1) * kArgmaxThreads < groups; g += UNROLL * kArgmaxThreads) {
            Vec<T> t[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) t[u].v = __ldg(&xv[g + u * kArgmaxThreads].v);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                for (int e = 0; e < N; ++e) offer(t[u].get(e), lo + (g + u * kArgmaxThreads) * N + e);
        }
        for (; g < groups; g += kArgmaxThreads) {
            Vec<T> t;
            t.v = __ldg(&xv[g].v);
#pragma unroll
            for (int e = 0; e < N; ++e) offer(t.get(e), lo + g * N + e);
        }
        c = lo + groups * N;  // scalar tail of the last range
    }
    // (per thread the indices above ascend only within a thread's own sequence, which is all `offer` needs)
    for (int64_t cc = c + threadIdx.x; cc < hi; cc += kArgmaxThreads) {
        const uint32_t k = order_key(spk_to_float<T>(xr[cc]));
        Best cand{k, cc};
        if (mine.i == INT64_MAX || argmax_better(cand, mine)) mine = cand;
    }
    __shared__ uint32_t sk[kArgmaxThreads / 32];
    __shared__ int64_t si[kArgmaxThreads / 32];
    mine = warp_best(mine, 32);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sk[warp] = mine.k; si[warp] = mine.i; }
    __syncthreads();
    if (warp == 0) {
        mine.k = lane < kArgmaxThreads / 32 ? sk[lane] : 0u;
        mine.i = lane < kArgmaxThreads / 32 ? si[lane] : INT64_MAX;
        mine = warp_best(mine, kArgmaxThreads / 32);
        if (lane == 0) {
            part_k[row * kArgmaxSplit + blockIdx.x] = mine.k;
            part_i[row * kArgmaxSplit + blockIdx.x] = mine.i;
        }
    }
}

// Pass 2: one warp per row folds the candidates.
__global__ void __launch_bounds__(32)
argmax_final_kernel(const uint32_t* __restrict__ part_k, const int64_t* __restrict__ part_i, int64_t* __restrict__ out) {
    const int64_t row = blockIdx.x;
    const int lane = threadIdx.x;
    Best mine{0u, INT64_MAX};
    if (lane < kArgmaxSplit) { mine.k = part_k[row * kArgmaxSplit + lane]; mine.i = part_i[row * kArgmaxSplit + lane]; }
    mine = warp_best(mine, 32);
    if (lane == 0) out[row] = mine.i == INT64_MAX ? 0 : mine.i;
}

}  // namespace

extern "C" int64_t spk_argmax_workspace_bytes(int64_t rows) {
    if (rows < 1) return 0;
    return rows * kArgmaxSplit * static_cast<int64_t>(sizeof(uint32_t) + sizeof(int64_t));
}

extern "C" int spk_argmax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int64_t* out,
                          void* workspace, int64_t workspace_bytes, void* stream) {
    SpkRange nvtx_range("spk_argmax");
    if (rows < 0 || cols < 1 || row_stride < cols) return SPK_ERR_BAD_SHAPE;
    if (dtype != SPK_F32 && dtype != SPK_BF16 && dtype != SPK_F16) return SPK_ERR_BAD_DTYPE;
    if (rows == 0) return SPK_OK;
    if (x == nullptr || out == nullptr) return SPK_ERR_NULL_POINTER;
    if (rows > 65535) return SPK_ERR_TOO_LARGE;
    if (workspace == nullptr || workspace_bytes < spk_argmax_workspace_bytes(rows)) return SPK_ERR_WORKSPACE_TOO_SMALL;
    // candidates: indices first (8-byte aligned at the start of the workspace), then keys
    int64_t* part_i = static_cast<int64_t*>(workspace);
    uint32_t* part_k = reinterpret_cast<uint32_t*>(part_i + rows * kArgmaxSplit);
    cudaStream_t s = spk_stream(stream);
    const dim3 grid(kArgmaxSplit, static_cast<unsigned>(rows));
    const int group = dtype == SPK_F32 ? 4 : 8;  // elements per 16 bytes
    const bool vec = reinterpret_cast<uintptr_t>(x) % 16 == 0 && row_stride % group == 0;
    int64_t per = (cols + kArgmaxSplit - 1) / kArgmaxSplit;
    per = (per + group - 1) / group * group;
#define SPK_ARGMAX(TX_)                                                                                      \
    do {                                                                                                     \
        if (vec) argmax_partial_kernel<TX_, true><<<grid, kArgmaxThreads, 0, s>>>(                           \
            static_cast<const TX_*>(x), row_stride, cols, per, part_k, part_i);                              \
        else argmax_partial_kernel<TX_, false><<<grid, kArgmaxThreads, 0, s>>>(                              \
            static_cast<const TX_*>(x), row_stride, cols, per, part_k, part_i);                              \
    } while (0)
    switch (dtype) {
        case SPK_F32: SPK_ARGMAX(float); break;
        case SPK_BF16: SPK_ARGMAX(__nv_bfloat16); break;
        default: SPK_ARGMAX(__half); break;
    }
#undef SPK_ARGMAX
    SPK_CHECK_LAUNCH();
    argmax_final_kernel<<<static_cast<unsigned>(rows), 32, 0, s>>>(part_k, part_i, out);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
