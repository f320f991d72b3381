// T-step leaky integrate-and-fire recurrence: dense-output kernel and the fused
// LIF + bit-pack + slot-mapped scatter kernel.
//
// Arithmetic contract (spikeinfer/kernels/lif_triton.py:13-28, :96-102 of the
// reference): the membrane is fp32 whatever the input type; beta is clamped to
// [0,1]; every step is ((beta*u) + I) - (r*theta) with each mul/add/sub rounded
// on its own (no FMA contraction: the __f*_rn intrinsics are never fused); the
// reset r is taken from the previous membrane; a spike is (u - theta) > 0, not
// u > theta.
#include "spk_common.cuh"

namespace {

__device__ __forceinline__ float clamp_beta(float b) {
    // Tensor.clamp(0, 1): NaN stays NaN.
    return b < 0.0f ? 0.0f : (b > 1.0f ? 1.0f : b);
}

// One neuron's state across timesteps.
struct Lif {
    float u;
    bool fired;  // H(u - theta) of the current membrane

    __device__ __forceinline__ void init(float u0, float th) {
        u = u0;
        fired = __fsub_rn(u, th) > 0.0f;
    }
    // Advances one step and returns the spike.
    template <int MODE>
    __device__ __forceinline__ bool step(float cur, float beta, float th) {
        if (MODE == SPK_RESET_SUBTRACT_DELAYED) {
            const float r = fired ? 1.0f : 0.0f;
            u = __fsub_rn(__fadd_rn(__fmul_rn(beta, u), cur), __fmul_rn(r, th));
            fired = __fsub_rn(u, th) > 0.0f;
            return fired;
        } else {
            u = __fadd_rn(__fmul_rn(beta, u), cur);
            const bool s = __fsub_rn(u, th) > 0.0f;
            if (s) u = 0.0f;
            fired = false;
            return s;
        }
    }
};

__device__ __forceinline__ void store_bit(void* base, int dtype, int64_t idx, bool b) {
    switch (dtype) {
        case SPK_F32: static_cast<float*>(base)[idx] = spk_bit_as<float>(b); break;
        case SPK_BF16: static_cast<__nv_bfloat16*>(base)[idx] = spk_bit_as<__nv_bfloat16>(b); break;
        case SPK_F16: static_cast<__half*>(base)[idx] = spk_bit_as<__half>(b); break;
        case SPK_U8: static_cast<uint8_t*>(base)[idx] = spk_bit_as<uint8_t>(b); break;
        default: static_cast<int32_t*>(base)[idx] = spk_bit_as<int32_t>(b); break;
    }
}

// ---------------------------------------------------------------------------
// Dense output: one thread per (row, channel), T steps in registers.
// ---------------------------------------------------------------------------
template <typename TX, int MODE>
__global__ void __launch_bounds__(256)
lif_dense_kernel(const TX* __restrict__ x, int T, int64_t stride_t, SpkDims mid, int64_t M,
                 int64_t N, const float* __restrict__ beta, const float* __restrict__ threshold,
                 const float* __restrict__ mem0, void* __restrict__ spikes, int spike_dtype,
                 float* __restrict__ mem_out) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= M * N) return;
    const int64_t m = idx / N;
    const int64_t n = idx - m * N;
    const float b = clamp_beta(beta[n]);
    const float th = threshold[n];
    const TX* xp = x + spk_row_offset(mid, m) + n;
    Lif s;
    s.init(mem0 != nullptr ? mem0[idx] : 0.0f, th);
    const int64_t plane = M * N;
    int t = 0;
    // Loads of four steps are issued together so their latencies overlap.
    for (; t + 4 <= T; t += 4) {
        float c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = spk_to_float<TX>(xp[(t + i) * stride_t]);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            store_bit(spikes, spike_dtype, (t + i) * plane + idx, s.template step<MODE>(c[i], b, th));
    }
    for (; t < T; ++t) {
        const float c = spk_to_float<TX>(xp[t * stride_t]);
        store_bit(spikes, spike_dtype, t * plane + idx, s.template step<MODE>(c, b, th));
    }
    if (mem_out != nullptr) mem_out[idx] = s.u;
}

// ---------------------------------------------------------------------------
// Fused LIF + pack + scatter.
//
// A warp owns kWordsPerWarp consecutive 32-channel words of one (token, head)
// row: lane i holds channel 32*w + i of each word, so a ballot of the spike
// predicate IS the packed word.  Timesteps are processed four at a time; the
// 4 * kWordsPerWarp ballots of a group are written by that many lanes, one
// word each.  K/V rows are redirected through slot_mapping on the way out.
// ---------------------------------------------------------------------------
constexpr int kWordsPerWarp = 2;
constexpr int kFusedThreads = 256;
constexpr int kStepGroup = 4;

struct SiteArgs {
    spk_lif_site s[SPK_MAX_LIF_SITES];
    int64_t warps[SPK_MAX_LIF_SITES];  // warps of work in each site
    int32_t groups[SPK_MAX_LIF_SITES]; // word groups per row
};

template <typename TX, int MODE>
__device__ __forceinline__ void fused_site(const spk_lif_site& s, int groups, int64_t warp, int lane,
                                           int T, int64_t n_tok, uint32_t* status) {
    const int64_t row = warp / groups;  // (tok, h)
    const int g = static_cast<int>(warp - row * groups);
    const int64_t tok = row / s.H;
    const int h = static_cast<int>(row - tok * s.H);
    const int64_t n_words = (s.N + 31) >> 5;
    const int w0 = g * kWordsPerWarp;

    const TX* xp = static_cast<const TX*>(s.x) + tok * s.sx_tok + h * s.sx_h;
    float b[kWordsPerWarp], th[kWordsPerWarp];
    bool live[kWordsPerWarp];
    Lif st[kWordsPerWarp];
#pragma unroll
    for (int j = 0; j < kWordsPerWarp; ++j) {
        const int64_t c = static_cast<int64_t>(w0 + j) * 32 + lane;
        live[j] = c < s.N;
        b[j] = live[j] ? clamp_beta(s.beta[c]) : 0.0f;
        th[j] = live[j] ? s.threshold[c] : 1.0f;
        float u0 = 0.0f;
        if (live[j] && s.mem0 != nullptr) u0 = s.mem0[row * s.N + c];
        st[j].init(u0, th[j]);
    }

    int64_t out_row = tok;
    bool row_ok = true;
    if (s.packed != nullptr && s.slot_mapping != nullptr) {
        out_row = s.slot_mapping[tok];
        row_ok = out_row >= 0 && out_row < s.num_rows;
        if (!row_ok && lane == 0) spk_flag(status, SPK_STATUS_BAD_SLOT);
    }

    for (int t0 = 0; t0 < T; t0 += kStepGroup) {
        float cur[kStepGroup][kWordsPerWarp];
#pragma unroll
        for (int i = 0; i < kStepGroup; ++i) {
#pragma unroll
            for (int j = 0; j < kWordsPerWarp; ++j) {
                cur[i][j] = 0.0f;
                if (t0 + i < T && live[j])
                    cur[i][j] = spk_to_float<TX>(
                        xp[(t0 + i) * s.sx_t + static_cast<int64_t>(w0 + j) * 32 + lane]);
            }
        }
        uint32_t mine = 0;  // lane i*kWordsPerWarp + j keeps word (t0 + i, w0 + j)
#pragma unroll
        for (int i = 0; i < kStepGroup; ++i) {
#pragma unroll
            for (int j = 0; j < kWordsPerWarp; ++j) {
                bool spike = false;
                if (t0 + i < T) {
                    spike = st[j].template step<MODE>(cur[i][j], b[j], th[j]) && live[j];
                    if (s.dense != nullptr && live[j]) {
                        const int64_t c = static_cast<int64_t>(w0 + j) * 32 + lane;
                        store_bit(s.dense, s.dense_dtype,
                                  (t0 + i) * s.sd_t + tok * s.sd_tok + h * s.sd_h + c, spike);
                    }
                }
                const uint32_t word = __ballot_sync(0xffffffffu, spike);
                if (lane == i * kWordsPerWarp + j) mine = word;
            }
        }
        if (s.packed != nullptr && row_ok && lane < kStepGroup * kWordsPerWarp) {
            const int i = lane / kWordsPerWarp;
            const int j = lane - i * kWordsPerWarp;
            if (t0 + i < T && w0 + j < n_words)
                reinterpret_cast<uint32_t*>(s.packed)[(t0 + i) * s.so_t + out_row * s.so_tok +
                                                      h * s.so_h + w0 + j] = mine;
        }
    }
    if (s.mem_out != nullptr) {
#pragma unroll
        for (int j = 0; j < kWordsPerWarp; ++j) {
            const int64_t c = static_cast<int64_t>(w0 + j) * 32 + lane;
            if (live[j]) s.mem_out[row * s.N + c] = st[j].u;
        }
    }
}

template <int MODE>
__global__ void __launch_bounds__(kFusedThreads)
lif_pack_scatter_kernel(SiteArgs args, int T, int64_t n_tok, uint32_t* status) {
    const int site = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kFusedThreads + threadIdx.x) >> 5;
    if (warp >= args.warps[site]) return;
    const spk_lif_site& s = args.s[site];
    switch (s.x_dtype) {
        case SPK_F32: fused_site<float, MODE>(s, args.groups[site], warp, lane, T, n_tok, status); break;
        case SPK_BF16: fused_site<__nv_bfloat16, MODE>(s, args.groups[site], warp, lane, T, n_tok, status); break;
        default: fused_site<__half, MODE>(s, args.groups[site], warp, lane, T, n_tok, status); break;
    }
}

template <typename TX>
int launch_dense(const void* x, int T, int64_t stride_t, const SpkDims& mid, int64_t M, int64_t N,
                 const float* beta, const float* threshold, const float* mem0, void* spikes,
                 int spike_dtype, float* mem_out, int reset_mode, cudaStream_t stream) {
    const int64_t blocks = (M * N + 255) / 256;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    const unsigned g = static_cast<unsigned>(blocks);
    if (reset_mode == SPK_RESET_SUBTRACT_DELAYED)
        lif_dense_kernel<TX, SPK_RESET_SUBTRACT_DELAYED><<<g, 256, 0, stream>>>(
            static_cast<const TX*>(x), T, stride_t, mid, M, N, beta, threshold, mem0, spikes,
            spike_dtype, mem_out);
    else
        lif_dense_kernel<TX, SPK_RESET_HARD_ZERO><<<g, 256, 0, stream>>>(
            static_cast<const TX*>(x), T, stride_t, mid, M, N, beta, threshold, mem0, spikes,
            spike_dtype, mem_out);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace

extern "C" int spk_lif(const void* x, int x_dtype, int T, int64_t stride_t, int n_mid,
                       const int64_t* mid_sizes, const int64_t* mid_strides, int64_t N,
                       const float* beta, const float* threshold, const float* mem0, void* spikes,
                       int spike_dtype, float* mem_out, int reset_mode, void* stream) {
    if (T < 0 || N <= 0) return SPK_ERR_BAD_SHAPE;
    if (reset_mode != SPK_RESET_SUBTRACT_DELAYED && reset_mode != SPK_RESET_HARD_ZERO)
        return SPK_ERR_UNSUPPORTED;
    if (spk_dtype_size(spike_dtype) == 0) return SPK_ERR_BAD_DTYPE;
    SpkDims mid;
    int64_t M = 0;
    int rc = spk_fill_dims(&mid, n_mid, mid_sizes, mid_strides, &M);
    if (rc != SPK_OK) return rc;
    if (M == 0 || (T == 0 && mem_out == nullptr)) return SPK_OK;
    if (x == nullptr || beta == nullptr || threshold == nullptr) return SPK_ERR_NULL_POINTER;
    if (T > 0 && spikes == nullptr) return SPK_ERR_NULL_POINTER;
    cudaStream_t s = spk_stream(stream);
    switch (x_dtype) {
        case SPK_F32:
            return launch_dense<float>(x, T, stride_t, mid, M, N, beta, threshold, mem0, spikes,
                                       spike_dtype, mem_out, reset_mode, s);
        case SPK_BF16:
            return launch_dense<__nv_bfloat16>(x, T, stride_t, mid, M, N, beta, threshold, mem0,
                                               spikes, spike_dtype, mem_out, reset_mode, s);
        case SPK_F16:
            return launch_dense<__half>(x, T, stride_t, mid, M, N, beta, threshold, mem0, spikes,
                                        spike_dtype, mem_out, reset_mode, s);
        default:
            return SPK_ERR_BAD_DTYPE;
    }
}

extern "C" int spk_lif_pack_scatter(const spk_lif_site* sites, int n_sites, int T, int64_t n_tok,
                                    int reset_mode, uint32_t* status, void* stream) {
    if (sites == nullptr) return SPK_ERR_NULL_POINTER;
    if (n_sites < 1 || n_sites > SPK_MAX_LIF_SITES || T < 1 || n_tok < 0) return SPK_ERR_BAD_SHAPE;
    if (reset_mode != SPK_RESET_SUBTRACT_DELAYED && reset_mode != SPK_RESET_HARD_ZERO)
        return SPK_ERR_UNSUPPORTED;
    if (n_tok == 0) return SPK_OK;
    SiteArgs args;
    int64_t max_warps = 0;
    for (int i = 0; i < SPK_MAX_LIF_SITES; ++i) {
        args.warps[i] = 0;
        args.groups[i] = 1;
    }
    for (int i = 0; i < n_sites; ++i) {
        const spk_lif_site& s = sites[i];
        if (s.x == nullptr || s.beta == nullptr || s.threshold == nullptr) return SPK_ERR_NULL_POINTER;
        if (s.x_dtype != SPK_F32 && s.x_dtype != SPK_BF16 && s.x_dtype != SPK_F16)
            return SPK_ERR_BAD_DTYPE;
        if (s.H < 1 || s.N < 1) return SPK_ERR_BAD_SHAPE;
        if (s.dense != nullptr && spk_dtype_size(s.dense_dtype) == 0) return SPK_ERR_BAD_DTYPE;
        if (s.packed != nullptr && s.slot_mapping != nullptr && s.num_rows < 1) return SPK_ERR_BAD_SHAPE;
        const int64_t words = (s.N + 31) / 32;
        const int64_t groups = (words + kWordsPerWarp - 1) / kWordsPerWarp;
        if (groups > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
        args.s[i] = s;
        args.groups[i] = static_cast<int32_t>(groups);
        args.warps[i] = n_tok * s.H * groups;
        if (args.warps[i] > max_warps) max_warps = args.warps[i];
    }
    const int warps_per_block = kFusedThreads / 32;
    const int64_t blocks = (max_warps + warps_per_block - 1) / warps_per_block;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(n_sites));
    cudaStream_t st = spk_stream(stream);
    if (reset_mode == SPK_RESET_SUBTRACT_DELAYED)
        lif_pack_scatter_kernel<SPK_RESET_SUBTRACT_DELAYED><<<grid, kFusedThreads, 0, st>>>(args, T, n_tok, status);
    else
        lif_pack_scatter_kernel<SPK_RESET_HARD_ZERO><<<grid, kFusedThreads, 0, st>>>(args, T, n_tok, status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
