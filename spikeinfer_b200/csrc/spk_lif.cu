// T-step leaky integrate-and-fire recurrence: dense-output kernel and the fused
// LIF + bit-pack + slot-mapped scatter kernel.
//
// Arithmetic contract (spikeinfer/kernels/lif_triton.py:13-28, :96-102 of the
// reference): the membrane is fp32 whatever the input type; beta is clamped to
// [0,1]; every step is ((beta*u) + I) - (r*theta) with each mul/add/sub rounded
// on its own (no FMA contraction: the __f*_rn intrinsics are never fused); the
// reset r is taken from the previous membrane; a spike is (u - theta) > 0 (see the
// note at struct Lif on why comparing u > theta directly is the same predicate here).
#include <utility>

#include "spk_common.cuh"

namespace {

__device__ __forceinline__ float clamp_beta(float b) {
    // Tensor.clamp(0, 1): NaN stays NaN.
    return b < 0.0f ? 0.0f : (b > 1.0f ? 1.0f : b);
}

// One neuron's state across timesteps.
//
// The spike predicate of the reference is (u - theta) > 0.  In IEEE arithmetic without flush-to-zero (this
// library is built without -ftz) a difference rounds to zero only when its operands are equal, and it is NaN
// exactly when the comparison is unordered, so (u - theta) > 0 and u > theta are the same predicate; the
// step below therefore compares directly and saves the subtraction.  The reset term r * theta is kept as
// "theta or 0" (1.0f * theta == theta and 0.0f * theta == 0 exactly for every finite theta).  The step is
// written in PTX so that the predicate is consumed by the next two instructions: with 8 channels in flight
// per lane, longer-lived predicates overflow the 7 predicate registers and cost a select + compare each.
struct Lif {
    float u;
    float rth;

    __device__ __forceinline__ void init(float u0, float th) {
        u = u0;
        rth = u > th ? th : 0.0f;
    }
    // Advances one step; ORs `bit` into `bits` when the neuron spikes.
    template <int MODE>
    __device__ __forceinline__ void step(float cur, float beta, float th, uint32_t bit, uint32_t& bits) {
        if (MODE == SPK_RESET_SUBTRACT_DELAYED) {
            asm("{\n\t.reg .pred p;\n\t"
                "mul.rn.f32 %0, %3, %0;\n\t"
                "add.rn.f32 %0, %0, %4;\n\t"
                "sub.rn.f32 %0, %0, %1;\n\t"
                "setp.gt.f32 p, %0, %5;\n\t"
                "selp.f32 %1, %5, 0f00000000, p;\n\t"
                "@p or.b32 %2, %2, %6;\n\t}"
                : "+f"(u), "+f"(rth), "+r"(bits)
                : "f"(beta), "f"(cur), "f"(th), "r"(bit));
        } else {
            asm("{\n\t.reg .pred p;\n\t"
                "mul.rn.f32 %0, %2, %0;\n\t"
                "add.rn.f32 %0, %0, %3;\n\t"
                "setp.gt.f32 p, %0, %4;\n\t"
                "@p mov.f32 %0, 0f00000000;\n\t"
                "@p or.b32 %1, %1, %5;\n\t}"
                : "+f"(u), "+r"(bits)
                : "f"(beta), "f"(cur), "f"(th), "r"(bit));
        }
    }
    // Same step with the spike's bit as an immediate operand (no register holds the constant).
    template <int MODE, uint32_t BIT>
    __device__ __forceinline__ void step_bit(float cur, float beta, float th, uint32_t& bits) {
        if (MODE == SPK_RESET_SUBTRACT_DELAYED) {
            asm("{\n\t.reg .pred p;\n\t"
                "mul.rn.f32 %0, %3, %0;\n\t"
                "add.rn.f32 %0, %0, %4;\n\t"
                "sub.rn.f32 %0, %0, %1;\n\t"
                "setp.gt.f32 p, %0, %5;\n\t"
                "selp.f32 %1, %5, 0f00000000, p;\n\t"
                "@p or.b32 %2, %2, %6;\n\t}"
                : "+f"(u), "+f"(rth), "+r"(bits)
                : "f"(beta), "f"(cur), "f"(th), "n"(BIT));
        } else {
            asm("{\n\t.reg .pred p;\n\t"
                "mul.rn.f32 %0, %2, %0;\n\t"
                "add.rn.f32 %0, %0, %3;\n\t"
                "setp.gt.f32 p, %0, %4;\n\t"
                "@p mov.f32 %0, 0f00000000;\n\t"
                "@p or.b32 %1, %1, %5;\n\t}"
                : "+f"(u), "+r"(bits)
                : "f"(beta), "f"(cur), "f"(th), "n"(BIT));
        }
    }
    template <int MODE>
    __device__ __forceinline__ bool step(float cur, float beta, float th) {
        uint32_t b = 0;
        step<MODE>(cur, beta, th, 1u, b);
        return b != 0;
    }
};

// Four timesteps of ONE channel from a zero membrane, channel-major: the spike predicate of a step is consumed by
// the next step's reset directly (`@p sub` / `@p mov`), so it lives for a handful of instructions and no register
// holds a reset term.  Same values as four Lif::step calls after init(0, th): u - 0 = u exactly, and the first
// step's beta * 0 + x is x + 0 for the finite beta >= 0 that clamp_beta guarantees.  Five instructions per
// element-step (four in the first) against six.
template <int MODE, uint32_t BIT>
__device__ __forceinline__ float lif_chain4(float x0, float x1, float x2, float x3, float beta, float th,
                                            uint32_t& b0, uint32_t& b1, uint32_t& b2, uint32_t& b3) {
    float u;
    if (MODE == SPK_RESET_SUBTRACT_DELAYED) {
        asm("{\n\t.reg .pred p;\n\t"
            "setp.gt.f32 p, 0f00000000, %6;\n\t"
            "add.rn.f32 %0, %7, 0f00000000;\n\t"
            "@p sub.rn.f32 %0, %0, %6;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %1, %1, %11;\n\t"
            "mul.rn.f32 %0, %5, %0;\n\t"
            "add.rn.f32 %0, %0, %8;\n\t"
            "@p sub.rn.f32 %0, %0, %6;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %2, %2, %11;\n\t"
            "mul.rn.f32 %0, %5, %0;\n\t"
            "add.rn.f32 %0, %0, %9;\n\t"
            "@p sub.rn.f32 %0, %0, %6;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %3, %3, %11;\n\t"
            "mul.rn.f32 %0, %5, %0;\n\t"
            "add.rn.f32 %0, %0, %10;\n\t"
            "@p sub.rn.f32 %0, %0, %6;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %4, %4, %11;\n\t}"
            : "=&f"(u), "+r"(b0), "+r"(b1), "+r"(b2), "+r"(b3)
            : "f"(beta), "f"(th), "f"(x0), "f"(x1), "f"(x2), "f"(x3), "n"(BIT));
    } else {
        asm("{\n\t.reg .pred p;\n\t"
            "add.rn.f32 %0, %7, 0f00000000;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %1, %1, %11;\n\t"
            "@p mov.f32 %0, 0f00000000;\n\t"
            "mul.rn.f32 %0, %5, %0;\n\t"
            "add.rn.f32 %0, %0, %8;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %2, %2, %11;\n\t"
            "@p mov.f32 %0, 0f00000000;\n\t"
            "mul.rn.f32 %0, %5, %0;\n\t"
            "add.rn.f32 %0, %0, %9;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %3, %3, %11;\n\t"
            "@p mov.f32 %0, 0f00000000;\n\t"
            "mul.rn.f32 %0, %5, %0;\n\t"
            "add.rn.f32 %0, %0, %10;\n\t"
            "setp.gt.f32 p, %0, %6;\n\t"
            "@p or.b32 %4, %4, %11;\n\t"
            "@p mov.f32 %0, 0f00000000;\n\t}"
            : "=&f"(u), "+r"(b0), "+r"(b1), "+r"(b2), "+r"(b3)
            : "f"(beta), "f"(th), "f"(x0), "f"(x1), "f"(x2), "f"(x3), "n"(BIT));
    }
    return u;
}

// ORs the bytes of the four lanes that build one packed word (lane & 3 = byte position) into every one of
// them.  A shuffle under a mask that differs between lanes is expanded by the compiler into a match/vote loop
// over the distinct masks (measured: ~7 of 17.8 instructions per element of the fused kernel), so a warp whose
// lanes are all live -- every warp but the edge ones -- shuffles under the full mask; `all_live` must be
// warp-uniform.  Otherwise only the group's own lanes take part (dead groups have left the loop body).
__device__ __forceinline__ uint32_t gather_word(uint32_t word, bool all_live, unsigned group_mask) {
    if (all_live) {
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
    } else {
        word |= __shfl_xor_sync(group_mask, word, 1);
        word |= __shfl_xor_sync(group_mask, word, 2);
    }
    return word;
}

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


constexpr int kFusedThreads = 256;
constexpr int kStepGroup = 4;

// ---------------------------------------------------------------------------
// Vectorised fused kernel (the fast path).
//
// A lane owns one segment of 8 consecutive channels of one (token, head) row and
// reads it with a single 16-byte load per timestep (two for fp32 inputs); the
// loads of four timesteps are in flight together.  Its 8 spike bits per timestep
// form one byte; the four lanes of a word exchange bytes with two xor-shuffles
// and the lane whose index matches the timestep writes the 32-bit word, so every
// lane issues exactly one word store per group of four timesteps.  Dense spikes
// and the membrane leave as 16/32-byte stores.  Requires N % 32 == 0 and
// 16-byte-aligned rows; anything else takes the ballot kernel below.
// ---------------------------------------------------------------------------
constexpr int kSeg = 8;

template <typename TX>
struct Raw8;
template <>
struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = __ldg(reinterpret_cast<const float4*>(p));
        b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    }
    __device__ __forceinline__ void from_smem(const uint4* p) {  // two pieces, 32 lanes apart
        a = *reinterpret_cast<const float4*>(p);
        b = *reinterpret_cast<const float4*>(p + 32);
    }
    __device__ __forceinline__ void clear() { a = make_float4(0, 0, 0, 0); b = a; }
    __device__ __forceinline__ float get(int i) const {
        switch (i) {
            case 0: return a.x; case 1: return a.y; case 2: return a.z; case 3: return a.w;
            case 4: return b.x; case 5: return b.y; case 6: return b.z; default: return b.w;
        }
    }
};
template <>
struct Raw8<__nv_bfloat16> {
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = __ldg(reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void from_smem(const uint4* p) { v = *p; }
    __device__ __forceinline__ void clear() { v = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
        // bf16 -> fp32 is exact: the 16 bits become the high half of the float
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
};
template <>
struct Raw8<__half> {
    uint4 v;
    __device__ __forceinline__ void load(const __half* p) { v = __ldg(reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void from_smem(const uint4* p) { v = *p; }
    __device__ __forceinline__ void clear() { v = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ float get(int i) const {
        const uint32_t w = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
        return __half2float(__ushort_as_half(static_cast<unsigned short>((i & 1) ? (w >> 16) : (w & 0xffffu))));
    }
};


// Four timesteps of the 8 channels of a segment, channel by channel; bit c of bits[t] = spike of channel c at t.
template <int MODE, typename TX, int... C>
__device__ __forceinline__ void chain8(const Raw8<TX> (&raw)[4], const float (&b)[8], const float (&th)[8],
                                       float (&u)[8], uint32_t (&bits)[4], std::integer_sequence<int, C...>) {
    ((u[C] = lif_chain4<MODE, (1u << C)>(raw[0].get(C), raw[1].get(C), raw[2].get(C), raw[3].get(C), b[C], th[C],
                                          bits[0], bits[1], bits[2], bits[3])), ...);
}

// The same with the currents supplied by `cur(t, channel)` (e.g. rotated on the fly).
template <int MODE, typename F, int... C>
__device__ __forceinline__ void chain8_of(F&& cur, const float (&b)[8], const float (&th)[8], float (&u)[8],
                                          uint32_t (&bits)[4], std::integer_sequence<int, C...>) {
    ((u[C] = lif_chain4<MODE, (1u << C)>(cur(0, C), cur(1, C), cur(2, C), cur(3, C), b[C], th[C], bits[0], bits[1],
                                          bits[2], bits[3])), ...);
}

// One timestep of the 8 channels of a segment; bit c of `bits` = spike of channel c.
template <int MODE, typename TX, int... C>
__device__ __forceinline__ void step8(Lif (&st)[8], const Raw8<TX>& raw, const float (&b)[8], const float (&th)[8],
                                      uint32_t& bits, std::integer_sequence<int, C...>) {
    (st[C].template step_bit<MODE, (1u << C)>(raw.get(C), b[C], th[C], bits), ...);
}

// Rounds an fp32 value to the element type TX and back (what a torch elementwise op in that dtype does).
template <typename TX>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }

// Packs 8 fp32 values (already representable in TX) into the 16/32 bytes of a dense TX row segment.
template <typename TX>
__device__ __forceinline__ void store8(TX* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (__float_as_uint(v[2 * i]) >> 16) | (__float_as_uint(v[2 * i + 1]) & 0xffff0000u);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        w[i] = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(v[2 * i]))) |
               (static_cast<uint32_t>(__half_as_ushort(__float2half_rn(v[2 * i + 1]))) << 16);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Writes 8 spikes (bit i of `bits` = channel i of the segment) as 0/1 in the dense type.
__device__ __forceinline__ void store_dense8(void* base, int dtype, int64_t idx, uint32_t bits) {
    if (dtype == SPK_BF16 || dtype == SPK_F16) {
        const uint32_t one = dtype == SPK_BF16 ? 0x3f80u : 0x3c00u;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = ((bits >> (2 * i)) & 1u ? one : 0u) | ((bits >> (2 * i + 1)) & 1u ? one << 16 : 0u);
        *reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if (dtype == SPK_F32) {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(base) + idx);
        o[0] = make_float4(bits & 1u ? 1.f : 0.f, bits & 2u ? 1.f : 0.f, bits & 4u ? 1.f : 0.f, bits & 8u ? 1.f : 0.f);
        o[1] = make_float4(bits & 16u ? 1.f : 0.f, bits & 32u ? 1.f : 0.f, bits & 64u ? 1.f : 0.f, bits & 128u ? 1.f : 0.f);
    } else if (dtype == SPK_U8) {
        // spread 8 bits into 8 bytes
        const uint32_t lo = ((bits & 0xfu) * 0x00204081u) & 0x01010101u;
        const uint32_t hi = (((bits >> 4) & 0xfu) * 0x00204081u) & 0x01010101u;
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(base) + idx) = make_uint2(lo, hi);
    } else {
        int4* o = reinterpret_cast<int4*>(static_cast<int32_t*>(base) + idx);
        o[0] = make_int4(bits & 1u, (bits >> 1) & 1u, (bits >> 2) & 1u, (bits >> 3) & 1u);
        o[1] = make_int4((bits >> 4) & 1u, (bits >> 5) & 1u, (bits >> 6) & 1u, (bits >> 7) & 1u);
    }
}

struct VecArgs {
    spk_lif_site s[SPK_MAX_LIF_SITES];
    uint32_t units[SPK_MAX_LIF_SITES];    // lanes of work in each site = token groups * per_tok
    uint32_t per_tok[SPK_MAX_LIF_SITES];  // segments per token = H * per_row
    uint32_t per_row[SPK_MAX_LIF_SITES];  // segments per (token, head) row = N / 8
    int32_t toks;                          // consecutive tokens a lane walks (amortises the parameter loads)
    int32_t slots;                         // 16-byte slots per lane and stage in the streaming form
};

// Asynchronous 16-byte global -> shared copy (per-thread completion groups).
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kStages = 3;  // tokens in flight per lane in the streaming form

// ASYNC (the streaming form for bandwidth-sized launches): a lane walks `toks` tokens and keeps the
// currents (and multiplicands) of the next kStages-1 tokens in flight with cp.async into its own slots
// of shared memory, so the bytes in flight per SM no longer depend on how many registers a warp holds.
// Every lane reads back only what it copied itself, so no barrier is involved.  Needs T <= 4, no RoPE.
// PLAIN: the site has no initial membrane, dense output, gated product or rotary embedding (checked on the
// host); the feature tests below then fold away at compile time.
template <typename TX, int MODE, bool ROPE, bool FULL, bool ASYNC, bool PLAIN>
__device__ __forceinline__ void fused_site_vec(const spk_lif_site& s, uint32_t units, uint32_t per_tok,
                                               uint32_t per_row, int toks, uint32_t unit, int lane, int T,
                                               int64_t n_tok, uint32_t* status, uint4* stage, int slots) {
    // 32-bit index arithmetic only: one lane = (token group, head, 8-channel segment)
    const bool in_range = unit < units;
    const uint32_t u_ = in_range ? unit : 0u;
    const uint32_t grp = u_ / per_tok;
    const uint32_t idx = u_ - grp * per_tok;
    const uint32_t h = s.H == 1 ? 0u : idx / per_row;
    const uint32_t sg = idx - h * per_row;
    const int c0 = static_cast<int>(sg) * kSeg;

    float b[kSeg], th[kSeg];
    {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(s.beta + c0));
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(s.beta + c0) + 1);
        const float4 t0 = __ldg(reinterpret_cast<const float4*>(s.threshold + c0));
        const float4 t1 = __ldg(reinterpret_cast<const float4*>(s.threshold + c0) + 1);
        const float bb[kSeg] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const float tt[kSeg] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
        for (int i = 0; i < kSeg; ++i) {
            b[i] = clamp_beta(bb[i]);
            th[i] = tt[i];
        }
    }
    const int sub = lane & 3;  // position of this lane's byte within its word
    // rotary embedding: channel c pairs with c + N/2 (first half, negated partner) or c - N/2 (second half)
    const bool rope = ROPE && s.rope_cos != nullptr;
    const bool first_half = 2 * sg < per_row;
    const int64_t partner_off = first_half ? s.N / 2 : -(s.N / 2);
    const float partner_sign = first_half ? -1.0f : 1.0f;

    // Site fields used in the loops, read once.
    const int64_t sx_t = s.sx_t, so_t = s.so_t, sd_t = s.sd_t, sm_t = s.sm_t, sg_t = s.sg_t, N = s.N;
    const bool has_packed = s.packed != nullptr, has_dense = !PLAIN && s.dense != nullptr;
    // the plain streaming form has no slots for the multiplicand, and the plain rotary form is the q/k/v launch
    const bool has_gated = !(PLAIN && (ASYNC || ROPE)) && s.gated != nullptr;
    const unsigned group_mask = 0xFu << (lane & 28);  // the four lanes that build one word together
    // byte selectors of the two exchange rounds of the 4 x 4 byte transpose (streaming plain form)
    const uint32_t sel_a = (lane & 1) ? 0x3715u : 0x6240u;  // even lane keeps timesteps 0 and 2 of its pair, odd 1 and 3
    const uint32_t sel_b = (lane & 2) ? 0x3276u : 0x5410u;  // then the lower pair keeps the lower timestep

    constexpr int VECS = sizeof(TX) * kSeg / 16;  // 16-byte pieces of one 8-channel segment
    auto issue = [&](int jj) {
        const int64_t tk = static_cast<int64_t>(grp) * toks + jj;
        if (jj < toks && in_range && tk < n_tok) {
            uint4* dst = stage + (jj % kStages) * slots * 32;
            const TX* xj = static_cast<const TX*>(s.x) + tk * s.sx_tok + static_cast<int64_t>(h) * s.sx_h + c0;
#pragma unroll
            for (int i = 0; i < kStepGroup; ++i) {
                if (FULL || i < T) {
#pragma unroll
                    for (int v = 0; v < VECS; ++v) cp_async16(dst + (i * VECS + v) * 32, xj + i * sx_t + v * (16 / sizeof(TX)));
                }
            }
            if (has_gated) {
                const TX* mj = static_cast<const TX*>(s.mul) + tk * s.sm_tok + static_cast<int64_t>(h) * s.sm_h + c0;
#pragma unroll
                for (int i = 0; i < kStepGroup; ++i) {
                    if (FULL || i < T) {
#pragma unroll
                        for (int v = 0; v < VECS; ++v)
                            cp_async16(dst + ((kStepGroup + i) * VECS + v) * 32, mj + i * sm_t + v * (16 / sizeof(TX)));
                    }
                }
            }
        }
        cp_async_commit();
    };
    if (ASYNC) {
#pragma unroll
        for (int jj = 0; jj < kStages - 1; ++jj) issue(jj);
    }

    for (int j = 0; j < toks; ++j) {
        const int64_t tok = static_cast<int64_t>(grp) * toks + j;
        if (ASYNC) {
            issue(j + kStages - 1);
            cp_async_wait<kStages - 1>();  // this lane's copies for token j have landed
        }
        // The four lanes of a word share (token group, head, word), so they are live or dead together and a
        // dead group skips the token; the byte exchange (gather_word) then runs under the group's own mask.
        const bool live = in_range && tok < n_tok;
        const bool all_live = __all_sync(0xffffffffu, live);
        if (!live) continue;
        const int64_t row = tok * s.H + h;
        Lif st[kSeg];
        {
            float u0[kSeg] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (!PLAIN && s.mem0 != nullptr) {
                const float4 m0 = __ldg(reinterpret_cast<const float4*>(s.mem0 + row * N + c0));
                const float4 m1 = __ldg(reinterpret_cast<const float4*>(s.mem0 + row * N + c0) + 1);
                u0[0] = m0.x; u0[1] = m0.y; u0[2] = m0.z; u0[3] = m0.w;
                u0[4] = m1.x; u0[5] = m1.y; u0[6] = m1.z; u0[7] = m1.w;
            }
#pragma unroll
            for (int i = 0; i < kSeg; ++i) st[i].init(u0[i], th[i]);
        }
        int64_t out_row = tok;
        bool row_ok = true;
        if (has_packed && s.slot_mapping != nullptr) {
            out_row = s.slot_mapping[tok];
            row_ok = out_row >= 0 && out_row < s.num_rows;
            if (!row_ok && sg == 0) spk_flag(status, SPK_STATUS_BAD_SLOT);
        }
        const int64_t head = static_cast<int64_t>(h);
        const TX* xp = static_cast<const TX*>(s.x) + tok * s.sx_tok + head * s.sx_h + c0;
        const TX* mp = has_gated ? static_cast<const TX*>(s.mul) + tok * s.sm_tok + head * s.sm_h + c0 : nullptr;
        TX* gp = has_gated ? static_cast<TX*>(s.gated) + tok * s.sg_tok + head * s.sg_h + c0 : nullptr;
        int64_t dense_idx = tok * s.sd_tok + head * s.sd_h + c0;
        uint32_t* wp = has_packed && row_ok
            ? reinterpret_cast<uint32_t*>(s.packed) + out_row * s.so_tok + head * s.so_h + (sg >> 2) + sub * so_t
            : nullptr;
        // The rotary factors are loaded here but unpacked only where they are used: touching them now would make the
        // warp wait for this load before it has issued the loads of the currents.
        Raw8<TX> cr, sr;
        if (rope) {
            cr.load(static_cast<const TX*>(s.rope_cos) + tok * s.s_rope_tok + c0);
            sr.load(static_cast<const TX*>(s.rope_sin) + tok * s.s_rope_tok + c0);
        } else {
            cr.clear();
            sr.clear();
        }

        if (ASYNC && PLAIN && FULL) {
            // Streaming form, nothing but bits (and the final membrane) asked for: the four timesteps of the
            // token come out of this lane's shared-memory slots together and every channel runs its four steps
            // in one go (lif_chain4).  The 4 x 4 bytes (lane of the word x timestep) are then transposed across
            // the word's four lanes in two exchange rounds, so that lane `sub` ends up with timestep `sub`'s word.
            const uint4* mine_stage = stage + (j % kStages) * slots * 32;
            Raw8<TX> raw[kStepGroup];
#pragma unroll
            for (int i = 0; i < kStepGroup; ++i) raw[i].from_smem(mine_stage + i * VECS * 32);
            float uf[kSeg];
            uint32_t bits[kStepGroup] = {0, 0, 0, 0};
            chain8<MODE, TX>(raw, b, th, uf, bits, std::make_integer_sequence<int, kSeg>{});
#pragma unroll
            for (int c = 0; c < kSeg; ++c) st[c].u = uf[c];
            uint32_t mine = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
            if (all_live) {
                mine = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 1), sel_a);
                mine = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 2), sel_b);
            } else {
                mine = __byte_perm(mine, __shfl_xor_sync(group_mask, mine, 1), sel_a);
                mine = __byte_perm(mine, __shfl_xor_sync(group_mask, mine, 2), sel_b);
            }
            if (wp != nullptr) *wp = mine;
        } else if (ASYNC) {
            // Streaming form: one timestep at a time straight from this lane's shared-memory slots (T <= 4),
            // rolled loop: few live registers, small code.
            const uint4* mine_stage = stage + (j % kStages) * slots * 32;
            uint32_t mine = 0;
#pragma unroll 1
            for (int i = 0; i < kStepGroup; ++i) {
                uint32_t bits = 0;
                if (FULL || i < T) {
                    Raw8<TX> raw;
                    raw.from_smem(mine_stage + i * VECS * 32);
                    step8<MODE, TX>(st, raw, b, th, bits, std::make_integer_sequence<int, kSeg>{});
                    if (has_gated) {
                        Raw8<TX> m;
                        m.from_smem(mine_stage + (kStepGroup + i) * VECS * 32);
                        float g[kSeg];
#pragma unroll
                        for (int c = 0; c < kSeg; ++c) g[c] = (bits >> c) & 1u ? m.get(c) : 0.0f;
                        store8<TX>(gp + i * sg_t, g);
                    }
                    if (has_dense) store_dense8(s.dense, s.dense_dtype, dense_idx + i * sd_t, bits);
                }
                uint32_t word = bits << (8 * sub);
                word = gather_word(word, all_live, group_mask);
                if (sub == i) mine = word;
            }
            if (wp != nullptr && (FULL || sub < T)) *wp = mine;
        } else if (PLAIN && FULL) {
            // The same channel-major form for launches too small to stream: the four timesteps straight from global
            // memory (four independent 16-byte loads per lane), T a multiple of four.
            for (int t0 = 0; t0 < T; t0 += kStepGroup) {
                Raw8<TX> raw[kStepGroup], mulv[kStepGroup];
#pragma unroll
                for (int i = 0; i < kStepGroup; ++i) raw[i].load(xp + i * sx_t);
                if (has_gated) {
#pragma unroll
                    for (int i = 0; i < kStepGroup; ++i) mulv[i].load(mp + i * sm_t);
                }
                uint32_t bits[kStepGroup] = {0, 0, 0, 0};
                if (ROPE && rope) {
                    // rotary embedding on the fly (T = 4 only, checked on the host): every operation rounded to the
                    // model dtype, as the eager expression (x * cos) + (rotate_half(x) * sin) does
                    Raw8<TX> partner[kStepGroup];
#pragma unroll
                    for (int i = 0; i < kStepGroup; ++i) partner[i].load(xp + i * sx_t + partner_off);
                    float uf[kSeg];
                    chain8_of<MODE>([&](int t, int c) {
                        const float a = round_to<TX>(__fmul_rn(raw[t].get(c), cr.get(c)));
                        const float r = round_to<TX>(__fmul_rn(partner_sign * partner[t].get(c), sr.get(c)));
                        return round_to<TX>(__fadd_rn(a, r));
                    }, b, th, uf, bits, std::make_integer_sequence<int, kSeg>{});
#pragma unroll
                    for (int c = 0; c < kSeg; ++c) st[c].init(uf[c], th[c]);
                } else if (t0 == 0) {
                    float uf[kSeg];
                    chain8<MODE, TX>(raw, b, th, uf, bits, std::make_integer_sequence<int, kSeg>{});
                    // membrane after the fourth step; its pending reset (u > th) is what init derives
#pragma unroll
                    for (int c = 0; c < kSeg; ++c) st[c].init(uf[c], th[c]);
                } else {
#pragma unroll
                    for (int i = 0; i < kStepGroup; ++i)
                        step8<MODE, TX>(st, raw[i], b, th, bits[i], std::make_integer_sequence<int, kSeg>{});
                }
                if (has_gated) {
                    // gated[t, tok, h, c] = spike ? mul[t, tok, h, c] : 0   (the spike * up product)
#pragma unroll
                    for (int i = 0; i < kStepGroup; ++i) {
                        float g[kSeg];
#pragma unroll
                        for (int c = 0; c < kSeg; ++c) g[c] = (bits[i] >> c) & 1u ? mulv[i].get(c) : 0.0f;
                        store8<TX>(gp + i * sg_t, g);
                    }
                    mp += kStepGroup * sm_t;
                    gp += kStepGroup * sg_t;
                }
                if (has_packed) {  // the same for the whole site, so the exchange below stays warp-uniform
                    uint32_t mine = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
                    if (all_live) {
                        mine = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 1), sel_a);
                        mine = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 2), sel_b);
                    } else {
                        mine = __byte_perm(mine, __shfl_xor_sync(group_mask, mine, 1), sel_a);
                        mine = __byte_perm(mine, __shfl_xor_sync(group_mask, mine, 2), sel_b);
                    }
                    if (wp != nullptr) {
                        *wp = mine;
                        wp += kStepGroup * so_t;
                    }
                }
                xp += kStepGroup * sx_t;
            }
        } else
        for (int t0 = 0; t0 < T; t0 += kStepGroup) {
            Raw8<TX> raw[kStepGroup], partner[kStepGroup], mulv[kStepGroup];
#pragma unroll
            for (int i = 0; i < kStepGroup; ++i) {
                const bool on = FULL || t0 + i < T;
                if (!FULL) { raw[i].clear(); mulv[i].clear(); }
                if (on) raw[i].load(xp + i * sx_t);
                if (has_gated && on) mulv[i].load(mp + i * sm_t);
                if (rope) {
                    if (!FULL) partner[i].clear();
                    if (on) partner[i].load(xp + i * sx_t + partner_off);
                }
            }
            // The loads above are all in flight at once; the arithmetic below is a ROLLED loop over the group's
            // timesteps (the step's registers are picked by a switch).  A small launch runs this code once per
            // thread, so its duration is the time to fetch the instructions: unrolled, the q/k/v launch of a
            // decode step spent 7.7 stall cycles per issued instruction waiting for instructions (ncu).
            uint32_t mine = 0;
#pragma unroll 1
            for (int i = 0; i < kStepGroup; ++i) {
                uint32_t bits = 0;
                if (FULL || t0 + i < T) {
                    Raw8<TX> x_i, partner_i, mul_i;
                    switch (i) {
                        case 0: x_i = raw[0]; partner_i = partner[0]; mul_i = mulv[0]; break;
                        case 1: x_i = raw[1]; partner_i = partner[1]; mul_i = mulv[1]; break;
                        case 2: x_i = raw[2]; partner_i = partner[2]; mul_i = mulv[2]; break;
                        default: x_i = raw[3]; partner_i = partner[3]; mul_i = mulv[3]; break;
                    }
#pragma unroll
                    for (int c = 0; c < kSeg; ++c) {
                        float cur = x_i.get(c);
                        if (rope) {
                            // (x * cos) + (rotate_half(x) * sin), every operation rounded to the model dtype
                            const float a = round_to<TX>(__fmul_rn(cur, cr.get(c)));
                            const float r = round_to<TX>(__fmul_rn(partner_sign * partner_i.get(c), sr.get(c)));
                            cur = round_to<TX>(__fadd_rn(a, r));
                        }
                        st[c].template step<MODE>(cur, b[c], th[c], 1u << c, bits);
                    }
                    if (has_gated) {
                        // gated[t, tok, h, c] = spike ? mul[t, tok, h, c] : 0   (the spike * up product)
                        float g[kSeg];
#pragma unroll
                        for (int c = 0; c < kSeg; ++c) g[c] = (bits >> c) & 1u ? mul_i.get(c) : 0.0f;
                        store8<TX>(gp + i * sg_t, g);
                    }
                    if (has_dense) store_dense8(s.dense, s.dense_dtype, dense_idx + (t0 + i) * sd_t, bits);
                }
                uint32_t word = bits << (8 * sub);
                word = gather_word(word, all_live, group_mask);
                if (sub == i) mine = word;
            }
            if (wp != nullptr && (FULL || t0 + sub < T)) *wp = mine;
            xp += kStepGroup * sx_t;
            if (has_gated) { mp += kStepGroup * sm_t; gp += kStepGroup * sg_t; }
            if (wp != nullptr) wp += kStepGroup * so_t;
        }
        if (s.mem_out != nullptr) {
            float4* o = reinterpret_cast<float4*>(s.mem_out + row * N + c0);
            o[0] = make_float4(st[0].u, st[1].u, st[2].u, st[3].u);
            o[1] = make_float4(st[4].u, st[5].u, st[6].u, st[7].u);
        }
    }
}

// The streaming plain form on its own (T = 4, no rotary embedding, no initial membrane, dense spikes or gated
// product): the same copies, arithmetic and stores as fused_site_vec<.., ASYNC, PLAIN> would issue, with the
// per-token bookkeeping reduced to running pointers and 32-bit counters.  At 11 instructions per element-step that
// bookkeeping was 40 % of the issue slots of an issue-bound kernel.
template <typename TX, int MODE>
__device__ __forceinline__ void stream_plain_site(const spk_lif_site& s, uint32_t units, uint32_t per_tok,
                                                  uint32_t per_row, int toks, uint32_t unit, int lane, int64_t n_tok,
                                                  uint32_t* status, uint4* stage, int slots) {
    if (unit >= units) return;  // the lanes of a word (4 consecutive units) are in or out together: units % 4 == 0
    const uint32_t grp = unit / per_tok;
    const uint32_t idx = unit - grp * per_tok;
    const uint32_t h = s.H == 1 ? 0u : idx / per_row;
    const uint32_t sg = idx - h * per_row;
    const int c0 = static_cast<int>(sg) * kSeg;
    const int sub = lane & 3;
    const unsigned group_mask = 0xFu << (lane & 28);
    const uint32_t sel_a = (lane & 1) ? 0x3715u : 0x6240u;
    const uint32_t sel_b = (lane & 2) ? 0x3276u : 0x5410u;
    constexpr int VECS = sizeof(TX) * kSeg / 16;

    const int64_t tok0 = static_cast<int64_t>(grp) * toks;
    const int64_t left64 = n_tok - tok0;
    const int n_mine = left64 < toks ? static_cast<int>(left64 > 0 ? left64 : 0) : toks;  // tokens of this lane's walk
    const int64_t sx_tok = s.sx_tok, sx_t = s.sx_t, so_tok = s.so_tok;
    const TX* xi = static_cast<const TX*>(s.x) + tok0 * sx_tok + static_cast<int64_t>(h) * s.sx_h + c0;  // next token to copy
    const uint32_t stage_bytes = static_cast<uint32_t>(slots) * 32u * 16u;
    const uint32_t stage0 = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
    uint32_t fill = 0;  // byte offset of the stage the next copy goes to
    int issued = 0;
    auto issue = [&]() {
        if (issued < n_mine) {
            const TX* p0 = xi;
#pragma unroll
            for (int i = 0; i < kStepGroup; ++i) {
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    const uint32_t dst = stage0 + fill + static_cast<uint32_t>((i * VECS + v) * 32 * 16);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(p0 + v * (16 / sizeof(TX))));
                }
                p0 += sx_t;
            }
            xi += sx_tok;
        }
        ++issued;
        fill = fill == (kStages - 1) * stage_bytes ? 0u : fill + stage_bytes;
        cp_async_commit();
    };
#pragma unroll
    for (int jj = 0; jj < kStages - 1; ++jj) issue();

    // weights of this lane's 8 channels (after the first copies are on their way)
    float b[kSeg], th[kSeg];
    {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(s.beta + c0));
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(s.beta + c0) + 1);
        const float4 t0 = __ldg(reinterpret_cast<const float4*>(s.threshold + c0));
        const float4 t1 = __ldg(reinterpret_cast<const float4*>(s.threshold + c0) + 1);
        const float bb[kSeg] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const float tt[kSeg] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
        for (int i = 0; i < kSeg; ++i) {
            b[i] = clamp_beta(bb[i]);
            th[i] = tt[i];
        }
    }
    const bool scatter = s.packed != nullptr && s.slot_mapping != nullptr;
    const int64_t* slot_p = scatter ? s.slot_mapping + tok0 : nullptr;
    uint32_t* wbase = s.packed != nullptr
        ? reinterpret_cast<uint32_t*>(s.packed) + static_cast<int64_t>(h) * s.so_h + (sg >> 2) + sub * s.so_t
        : nullptr;
    uint32_t* wp = wbase != nullptr && !scatter ? wbase + tok0 * so_tok : nullptr;  // running, when rows are the tokens
    const int64_t mem_step = static_cast<int64_t>(s.H) * s.N;
    float* mo = s.mem_out != nullptr ? s.mem_out + (tok0 * s.H + h) * s.N + c0 : nullptr;
    uint32_t drain = 0;  // byte offset of the stage the next token is read from

    for (int j = 0; j < toks; ++j) {
        issue();
        cp_async_wait<kStages - 1>();  // this lane's copies for token j have landed
        const bool live = j < n_mine;
        const bool all_live = __all_sync(0xffffffffu, live);
        const uint4* mine_stage = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(stage) + drain);
        drain = drain == (kStages - 1) * stage_bytes ? 0u : drain + stage_bytes;
        if (!live) continue;
        Raw8<TX> raw[kStepGroup];
#pragma unroll
        for (int i = 0; i < kStepGroup; ++i) raw[i].from_smem(mine_stage + i * VECS * 32);
        float uf[kSeg];
        uint32_t bits[kStepGroup] = {0, 0, 0, 0};
        chain8<MODE, TX>(raw, b, th, uf, bits, std::make_integer_sequence<int, kSeg>{});
        uint32_t mine = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
        if (all_live) {
            mine = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 1), sel_a);
            mine = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 2), sel_b);
        } else {
            mine = __byte_perm(mine, __shfl_xor_sync(group_mask, mine, 1), sel_a);
            mine = __byte_perm(mine, __shfl_xor_sync(group_mask, mine, 2), sel_b);
        }
        if (scatter) {
            const int64_t out_row = slot_p[j];
            if (out_row >= 0 && out_row < s.num_rows) wbase[out_row * so_tok] = mine;
            else if (sg == 0) spk_flag(status, SPK_STATUS_BAD_SLOT);
        } else if (wp != nullptr) {
            *wp = mine;
            wp += so_tok;
        }
        if (mo != nullptr) {
            float4* o = reinterpret_cast<float4*>(mo);
            o[0] = make_float4(uf[0], uf[1], uf[2], uf[3]);
            o[1] = make_float4(uf[4], uf[5], uf[6], uf[7]);
            mo += mem_step;
        }
    }
}

template <int MODE, bool ROPE, bool FULL, bool ASYNC, bool PLAIN>
__global__ void __launch_bounds__(kFusedThreads, (ROPE && !PLAIN) ? 1 : (ASYNC ? 4 : 2))
lif_pack_scatter_vec_kernel(VecArgs args, int T, int64_t n_tok, uint32_t* status) {
    // A next launch that asked to overlap this one (the attention after the q/k/v sites: it reads only lengths and
    // block tables until this grid has finished) may be placed from now on; without such a launch this does nothing.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint4 stage_smem[];
    const int site = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const uint32_t unit = blockIdx.x * kFusedThreads + threadIdx.x;
    if (unit - lane >= args.units[site]) return;  // whole warp out of range
    const spk_lif_site& s = args.s[site];
    // this lane's slots: [warp][stage][slot][lane]
    uint4* stage = ASYNC ? stage_smem + (threadIdx.x >> 5) * kStages * args.slots * 32 + lane : nullptr;
#define SPK_SITE(TX_)                                                                                              \
    do {                                                                                                            \
        if (ASYNC && PLAIN && FULL && !ROPE)                                                                        \
            stream_plain_site<TX_, MODE>(s, args.units[site], args.per_tok[site], args.per_row[site], args.toks,    \
                                         unit, lane, n_tok, status, stage, args.slots);                             \
        else                                                                                                        \
            fused_site_vec<TX_, MODE, ROPE, FULL, ASYNC, PLAIN>(s, args.units[site], args.per_tok[site],            \
                                                                args.per_row[site], args.toks, unit, lane, T, n_tok, \
                                                                status, stage, args.slots);                         \
    } while (0)
    switch (s.x_dtype) {
        case SPK_F32: SPK_SITE(float); break;
        case SPK_BF16: SPK_SITE(__nv_bfloat16); break;
        default: SPK_SITE(__half); break;
    }
#undef SPK_SITE
}

static inline bool is_aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

// Can this site take the vectorised kernel?
static bool site_vectorisable(const spk_lif_site& s) {
    if (s.N % 32 != 0) return false;
    const int xs = spk_dtype_size(s.x_dtype);
    const int64_t xq = 16 / xs;  // elements per 16 bytes
    if (!is_aligned(s.x, 16) || s.sx_t % xq || s.sx_tok % xq || s.sx_h % xq) return false;
    if (!is_aligned(s.beta, 16) || !is_aligned(s.threshold, 16)) return false;
    if (s.mem0 != nullptr && !is_aligned(s.mem0, 16)) return false;
    if (s.mem_out != nullptr && !is_aligned(s.mem_out, 16)) return false;
    if (s.rope_cos != nullptr) {
        if (s.rope_sin == nullptr || !is_aligned(s.rope_cos, 16) || !is_aligned(s.rope_sin, 16) || s.s_rope_tok % xq)
            return false;
    }
    if (s.gated != nullptr) {
        if (s.mul == nullptr || !is_aligned(s.mul, 16) || !is_aligned(s.gated, 16)) return false;
        if (s.sm_t % xq || s.sm_tok % xq || s.sm_h % xq || s.sg_t % xq || s.sg_tok % xq || s.sg_h % xq) return false;
    }
    if (s.dense != nullptr) {
        const int ds = spk_dtype_size(s.dense_dtype);
        const int64_t bytes = ds == 1 ? 8 : 16;
        const int64_t dq = bytes / ds;
        if (!is_aligned(s.dense, bytes) || s.sd_t % dq || s.sd_tok % dq || s.sd_h % dq) return false;
    }
    return true;
}

// ---------------------------------------------------------------------------
// Fused LIF + pack + scatter, general (ballot) form.
//
// A warp owns kWordsPerWarp consecutive 32-channel words of one (token, head)
// row: lane i holds channel 32*w + i of each word, so a ballot of the spike
// predicate IS the packed word.  Timesteps are processed four at a time; the
// 4 * kWordsPerWarp ballots of a group are written by that many lanes, one
// word each.  K/V rows are redirected through slot_mapping on the way out.
// ---------------------------------------------------------------------------
constexpr int kWordsPerWarp = 2;

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
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see lif_pack_scatter_vec_kernel
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
    SpkRange nvtx_range("spk_lif");
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
    if (n_mid <= 2 && T > 0 && (x_dtype == SPK_F32 || x_dtype == SPK_BF16 || x_dtype == SPK_F16)) {
        // Rows addressable as (tok, h): use the vectorised kernel with a dense-only site.
        spk_lif_site site = {};
        site.x = x; site.x_dtype = x_dtype; site.N = N;
        const int64_t n_tok = n_mid >= 1 ? mid.size[0] : 1;
        site.H = static_cast<int32_t>(n_mid == 2 ? mid.size[1] : 1);
        site.sx_t = stride_t;
        site.sx_tok = n_mid >= 1 ? mid.stride[0] : 0;
        site.sx_h = n_mid == 2 ? mid.stride[1] : 0;
        site.beta = beta; site.threshold = threshold; site.mem0 = mem0; site.mem_out = mem_out;
        site.dense = spikes; site.dense_dtype = spike_dtype;
        site.sd_t = M * N; site.sd_tok = static_cast<int64_t>(site.H) * N; site.sd_h = N;
        if ((n_mid < 2 || mid.size[1] <= 0x7fffffffLL) && site_vectorisable(site))
            return spk_lif_pack_scatter(&site, 1, T, n_tok, reset_mode, nullptr, stream);
    }
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
    SpkRange nvtx_range("spk_lif_pack_scatter");
    if (sites == nullptr) return SPK_ERR_NULL_POINTER;
    if (n_sites < 1 || n_sites > SPK_MAX_LIF_SITES || T < 1 || n_tok < 0) return SPK_ERR_BAD_SHAPE;
    if (reset_mode != SPK_RESET_SUBTRACT_DELAYED && reset_mode != SPK_RESET_HARD_ZERO)
        return SPK_ERR_UNSUPPORTED;
    if (n_tok == 0) return SPK_OK;
    bool vec = true;
    for (int i = 0; i < n_sites; ++i) {
        const spk_lif_site& s = sites[i];
        if (s.x == nullptr || s.beta == nullptr || s.threshold == nullptr) return SPK_ERR_NULL_POINTER;
        if (s.x_dtype != SPK_F32 && s.x_dtype != SPK_BF16 && s.x_dtype != SPK_F16) return SPK_ERR_BAD_DTYPE;
        if (s.H < 1 || s.N < 1) return SPK_ERR_BAD_SHAPE;
        if (s.dense != nullptr && spk_dtype_size(s.dense_dtype) == 0) return SPK_ERR_BAD_DTYPE;
        if (s.packed != nullptr && s.slot_mapping != nullptr && s.num_rows < 1) return SPK_ERR_BAD_SHAPE;
        vec = vec && site_vectorisable(s);
    }
    if (vec) {
        VecArgs va;
        // tokens per lane: 4 once that still leaves every SM a few thousand lanes, else 2 or 1
        int64_t widest = 0;
        for (int i = 0; i < n_sites; ++i) widest = widest > sites[i].H * (sites[i].N / kSeg) ? widest : sites[i].H * (sites[i].N / kSeg);
        bool any_rope = false, any_gated = false, any_f32 = false;
        for (int i = 0; i < n_sites; ++i) {
            any_rope = any_rope || sites[i].rope_cos != nullptr;
            any_gated = any_gated || sites[i].gated != nullptr;
            any_f32 = any_f32 || sites[i].x_dtype == SPK_F32;
        }
        int toks = 4;
        while (toks > 1 && (n_tok / toks) * widest < 148LL * 2048) toks >>= 1;
        // Bandwidth-sized launches stream through shared memory (cp.async, kStages tokens in flight per lane).
        const bool streaming = !any_rope && T <= kStepGroup && toks == 4 && (n_tok / 8) * widest >= 148LL * 2048;
        if (streaming) toks = 8;
        va.toks = toks;
        va.slots = kStepGroup * (any_f32 ? 2 : 1) * (any_gated ? 2 : 1);
        const size_t stage_bytes = streaming ? static_cast<size_t>(kFusedThreads / 32) * kStages * va.slots * 32 * 16 : 0;
        const int64_t groups = (n_tok + toks - 1) / toks;
        int64_t max_units = 0;
        for (int i = 0; i < SPK_MAX_LIF_SITES; ++i) {
            va.units[i] = 0;
            va.per_tok[i] = 1;
            va.per_row[i] = 1;
        }
        bool fits = true;
        for (int i = 0; i < n_sites; ++i) {
            va.s[i] = sites[i];
            const int64_t per_row = sites[i].N / kSeg;
            const int64_t per_tok = per_row * sites[i].H;
            const int64_t units = groups * per_tok;
            if (units >= 0x7fffffffLL) fits = false;
            va.per_row[i] = static_cast<uint32_t>(per_row);
            va.per_tok[i] = static_cast<uint32_t>(per_tok);
            va.units[i] = static_cast<uint32_t>(units);
            if (units > max_units) max_units = units;
        }
        if (fits) {
            const int64_t vblocks = (max_units + kFusedThreads - 1) / kFusedThreads;
            dim3 vgrid(static_cast<unsigned>(vblocks), static_cast<unsigned>(n_sites));
            cudaStream_t vst = spk_stream(stream);
            const bool sub = reset_mode == SPK_RESET_SUBTRACT_DELAYED;
            const bool full = T % kStepGroup == 0;  // no partial group of timesteps: the per-step bounds checks drop out
            bool plain = true;  // packed bits, gated product, final membrane only: the other feature tests fold away
            for (int i = 0; i < n_sites; ++i) plain = plain && sites[i].mem0 == nullptr && sites[i].dense == nullptr;
            const bool plain_rope = plain && any_rope && !any_gated && T == kStepGroup;  // the decode step's q/k/v launch
            plain = plain && !any_rope;
#define SPK_LAUNCH_VEC(MODE_, ROPE_, FULL_, ASYNC_, PLAIN_)                                                                \
    do {                                                                                                              \
        auto kern = lif_pack_scatter_vec_kernel<MODE_, ROPE_, FULL_, ASYNC_, PLAIN_>;                                       \
        if (stage_bytes > 48 * 1024) {                                                                                \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                                                       static_cast<int>(stage_bytes));                                \
            if (e != cudaSuccess) return spk_set_cuda_error(e);                                                       \
        }                                                                                                             \
        kern<<<vgrid, kFusedThreads, stage_bytes, vst>>>(va, T, n_tok, status);                                       \
    } while (0)
#define SPK_LAUNCH_MODE(MODE_)                                                          \
    do {                                                                                \
        if (streaming && full && plain && !any_gated) SPK_LAUNCH_VEC(MODE_, false, true, true, true); \
        else if (streaming) { if (full) SPK_LAUNCH_VEC(MODE_, false, true, true, false); else SPK_LAUNCH_VEC(MODE_, false, false, true, false); } \
        else if (plain_rope) SPK_LAUNCH_VEC(MODE_, true, true, false, true); \
        else if (any_rope) { if (full) SPK_LAUNCH_VEC(MODE_, true, true, false, false); else SPK_LAUNCH_VEC(MODE_, true, false, false, false); } \
        else if (full && plain) SPK_LAUNCH_VEC(MODE_, false, true, false, true); \
        else { if (full) SPK_LAUNCH_VEC(MODE_, false, true, false, false); else SPK_LAUNCH_VEC(MODE_, false, false, false, false); } \
    } while (0)
            if (sub) SPK_LAUNCH_MODE(SPK_RESET_SUBTRACT_DELAYED);
            else SPK_LAUNCH_MODE(SPK_RESET_HARD_ZERO);
#undef SPK_LAUNCH_MODE
#undef SPK_LAUNCH_VEC
            SPK_CHECK_LAUNCH();
            return SPK_OK;
        }
    }
    for (int i = 0; i < n_sites; ++i) {
        // the rotary and gated-product fusions exist only in the vectorised kernel
        if (sites[i].rope_cos != nullptr || sites[i].gated != nullptr) return SPK_ERR_UNSUPPORTED;
    }
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
