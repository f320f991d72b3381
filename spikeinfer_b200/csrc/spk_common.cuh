// Shared helpers for the sm_100a spiking-decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/spikeinfer_b200.h"

#define SPK_MAX_DIMS 6

// Launch-error bookkeeping shared by all translation units (defined in spk_capi.cu).
int spk_set_cuda_error(cudaError_t err);

void spk_count_launch();

#define SPK_CHECK_LAUNCH()                               \
    do {                                                 \
        cudaError_t e__ = cudaGetLastError();            \
        if (e__ != cudaSuccess) return spk_set_cuda_error(e__); \
        spk_count_launch();                              \
    } while (0)

// NVTX range around an entry point's launches, for timelines taken with a profiler.  Off unless the
// environment holds SPK_NVTX=1 when the library makes its first call (defined in spk_capi.cu).
struct SpkRange {
    explicit SpkRange(const char* name);
    ~SpkRange();
    SpkRange(const SpkRange&) = delete;
    SpkRange& operator=(const SpkRange&) = delete;
    bool on;
};

static inline cudaStream_t spk_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Up to SPK_MAX_DIMS leading dimensions of a strided array, innermost last.
struct SpkDims {
    int n;
    int64_t size[SPK_MAX_DIMS];
    int64_t stride[SPK_MAX_DIMS];
};

// Offset (in elements) of flat row index `row` over the leading dimensions.
__device__ __forceinline__ int64_t spk_row_offset(const SpkDims& d, int64_t row) {
    int64_t off = 0;
#pragma unroll
    for (int i = SPK_MAX_DIMS - 1; i >= 0; --i) {
        if (i < d.n) {
            int64_t q = row / d.size[i];
            off += (row - q * d.size[i]) * d.stride[i];
            row = q;
        }
    }
    return off;
}

static inline int spk_fill_dims(SpkDims* d, int n, const int64_t* sizes, const int64_t* strides,
                                int64_t* rows_out) {
    if (n < 0 || n > SPK_MAX_DIMS) return SPK_ERR_BAD_SHAPE;
    if (n > 0 && (sizes == nullptr || strides == nullptr)) return SPK_ERR_NULL_POINTER;
    int64_t rows = 1;
    d->n = n;
    for (int i = 0; i < SPK_MAX_DIMS; ++i) {
        d->size[i] = 1;
        d->stride[i] = 0;
    }
    for (int i = 0; i < n; ++i) {
        if (sizes[i] < 0) return SPK_ERR_BAD_SHAPE;
        d->size[i] = sizes[i] > 0 ? sizes[i] : 1;
        d->stride[i] = strides[i];
        rows *= sizes[i];
    }
    *rows_out = rows;
    return SPK_OK;
}

// Exact widening loads: every supported input type converts to fp32 without rounding.
template <typename T>
__device__ __forceinline__ float spk_to_float(T v);
template <>
__device__ __forceinline__ float spk_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float spk_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float spk_to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float spk_to_float<uint8_t>(uint8_t v) { return static_cast<float>(v); }
template <>
__device__ __forceinline__ float spk_to_float<int32_t>(int32_t v) { return static_cast<float>(v); }

template <typename T>
__device__ __forceinline__ bool spk_nonzero(T v) { return v != static_cast<T>(0); }
template <>
__device__ __forceinline__ bool spk_nonzero<__nv_bfloat16>(__nv_bfloat16 v) {
    // +-0 are the only zeros; NaN counts as a spike, as (x != 0) does.
    return (__bfloat16_as_ushort(v) & 0x7fffu) != 0;
}
template <>
__device__ __forceinline__ bool spk_nonzero<__half>(__half v) {
    return (__half_as_ushort(v) & 0x7fffu) != 0;
}

// 0/1 in the requested element type.
template <typename T>
__device__ __forceinline__ T spk_bit_as(bool b);
template <>
__device__ __forceinline__ float spk_bit_as<float>(bool b) { return b ? 1.0f : 0.0f; }
template <>
__device__ __forceinline__ __nv_bfloat16 spk_bit_as<__nv_bfloat16>(bool b) {
    return __ushort_as_bfloat16(b ? 0x3f80u : 0u);
}
template <>
__device__ __forceinline__ __half spk_bit_as<__half>(bool b) {
    return __ushort_as_half(b ? 0x3c00u : 0u);
}
template <>
__device__ __forceinline__ uint8_t spk_bit_as<uint8_t>(bool b) { return b ? 1 : 0; }
template <>
__device__ __forceinline__ int32_t spk_bit_as<int32_t>(bool b) { return b ? 1 : 0; }

__device__ __forceinline__ void spk_flag(uint32_t* status, uint32_t bit) {
    if (status != nullptr) atomicOr(status, bit);
}

static inline int spk_dtype_size(int dtype) {
    switch (dtype) {
        case SPK_F32: return 4;
        case SPK_BF16: return 2;
        case SPK_F16: return 2;
        case SPK_U8: return 1;
        case SPK_I32: return 4;
        default: return 0;
    }
}
