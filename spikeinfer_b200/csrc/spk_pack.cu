// Bit packing / unpacking of spike tensors.
//
// Layout (spikeinfer/kernels/packing.py:15-23 of the reference): bit i of word w
// holds channel 32*w + i, words ascend along the channel axis, the unused tail of
// the last word is zero.  Words are int32 at the torch surface and uint32 here.
#include "spk_common.cuh"

namespace {

constexpr int kPackThreads = 256;

// One warp per (row, word): lane i tests channel 32*w + i, a ballot builds the word.
template <typename T>
__global__ void __launch_bounds__(kPackThreads)
pack_kernel(const T* __restrict__ x, SpkDims dims, int64_t rows, int64_t channels, int words,
            uint32_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kPackThreads + threadIdx.x) >> 5;
    const int64_t total = rows * words;
    if (warp >= total) return;
    const int64_t row = warp / words;
    const int w = static_cast<int>(warp - row * words);
    const int64_t c = static_cast<int64_t>(w) * 32 + lane;
    bool bit = false;
    if (c < channels) bit = spk_nonzero<T>(x[spk_row_offset(dims, row) + c]);
    const uint32_t word = __ballot_sync(0xffffffffu, bit);
    if (lane == 0) out[warp] = word;
}

template <typename T>
__global__ void __launch_bounds__(256)
unpack_kernel(const uint32_t* __restrict__ words, int64_t rows, int64_t channels, int n_words,
              T* __restrict__ out) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * channels) return;
    const int64_t row = idx / channels;
    const int c = static_cast<int>(idx - row * channels);
    const uint32_t word = words[row * n_words + (c >> 5)];
    out[idx] = spk_bit_as<T>((word >> (c & 31)) & 1u);
}

template <typename T>
int launch_pack(const void* x, const SpkDims& dims, int64_t rows, int64_t channels, int words,
                int32_t* out, cudaStream_t stream) {
    const int64_t warps = rows * words;
    const int64_t blocks = (warps * 32 + kPackThreads - 1) / kPackThreads;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    pack_kernel<T><<<static_cast<unsigned>(blocks), kPackThreads, 0, stream>>>(
        static_cast<const T*>(x), dims, rows, channels, words, reinterpret_cast<uint32_t*>(out));
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

template <typename T>
int launch_unpack(const int32_t* words, int64_t rows, int64_t channels, int n_words, void* out,
                  cudaStream_t stream) {
    const int64_t total = rows * channels;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    unpack_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint32_t*>(words), rows, channels, n_words, static_cast<T*>(out));
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace

extern "C" int spk_pack(const void* x, int x_dtype, int ndim, const int64_t* sizes,
                        const int64_t* strides, int64_t channels, int32_t* out, void* stream) {
    if (channels <= 0) return SPK_ERR_BAD_SHAPE;
    SpkDims dims;
    int64_t rows = 0;
    int rc = spk_fill_dims(&dims, ndim, sizes, strides, &rows);
    if (rc != SPK_OK) return rc;
    if (rows == 0) return SPK_OK;
    if (x == nullptr || out == nullptr) return SPK_ERR_NULL_POINTER;
    const int64_t words = (channels + 31) / 32;
    if (words > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    cudaStream_t s = spk_stream(stream);
    switch (x_dtype) {
        case SPK_F32: return launch_pack<float>(x, dims, rows, channels, (int)words, out, s);
        case SPK_BF16: return launch_pack<__nv_bfloat16>(x, dims, rows, channels, (int)words, out, s);
        case SPK_F16: return launch_pack<__half>(x, dims, rows, channels, (int)words, out, s);
        case SPK_U8: return launch_pack<uint8_t>(x, dims, rows, channels, (int)words, out, s);
        case SPK_I32: return launch_pack<int32_t>(x, dims, rows, channels, (int)words, out, s);
        default: return SPK_ERR_BAD_DTYPE;
    }
}

extern "C" int spk_unpack(const int32_t* words, int64_t rows, int64_t channels, void* out,
                          int out_dtype, void* stream) {
    if (channels <= 0 || rows < 0) return SPK_ERR_BAD_SHAPE;
    if (rows == 0) return SPK_OK;
    if (words == nullptr || out == nullptr) return SPK_ERR_NULL_POINTER;
    const int64_t n_words = (channels + 31) / 32;
    if (n_words > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    cudaStream_t s = spk_stream(stream);
    switch (out_dtype) {
        case SPK_F32: return launch_unpack<float>(words, rows, channels, (int)n_words, out, s);
        case SPK_BF16: return launch_unpack<__nv_bfloat16>(words, rows, channels, (int)n_words, out, s);
        case SPK_F16: return launch_unpack<__half>(words, rows, channels, (int)n_words, out, s);
        case SPK_U8: return launch_unpack<uint8_t>(words, rows, channels, (int)n_words, out, s);
        case SPK_I32: return launch_unpack<int32_t>(words, rows, channels, (int)n_words, out, s);
        default: return SPK_ERR_BAD_DTYPE;
    }
}
