// Paged popcount decode attention over bit-packed spike K/V.
//
// out[t,n,h,:] = softmax_j( popc(q[t,n,h] & k_j) * scale ) . v_j   over the keys of sequence n
// (spikeinfer/kernels/spike_attention.py:67-150 of the reference).
//
// Formulation used here:
//  * A warp owns one work item = (sequence, timestep, KV head, key range) and serves all query
//    heads of the GQA group from a single read of K and V.
//  * popc(q & k) <= popc(q), so the softmax is taken against the fixed bound m = popc(q)*scale
//    instead of a running maximum.  That is the same softmax (a common factor cancels), it cannot
//    overflow, and the smallest weight, exp(-head_dim*scale), is far above fp32 underflow.  Partial
//    sums of different key ranges therefore combine by plain addition.
//  * A score is an integer in [0, popc(q)], so a weight takes at most head_dim+1 values: they come
//    from a per-item table in shared memory, indexed by the exact integer score.
//  * Phase A (lane = key): coalesced K/V row loads, scores with __popc, weights from the table,
//    staged to shared memory together with the V words.
//    Phase B (lane = channel group): every staged key is broadcast; a lane adds the key's weight to
//    the accumulators of the channels whose V bit is set ("bit-selected sum"), fp32.
//  * No tensor cores: the operands are 1-bit and the contraction is a conditional add.
#include "spk_common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kStageWords = 12;  // [w0..w3][w4..w7][v0..v3]
constexpr int kMaxSplits = 256;
constexpr int kTargetWarps = 148 * 4 * 4;  // four warps per scheduler

struct AttnParams {
    const uint32_t* q; int64_t sq_t, sq_n, sq_h;
    const uint32_t* k; int64_t sk_t, sk_h, sk_blk, sk_slot;
    const uint32_t* v; int64_t sv_t, sv_h, sv_blk, sv_slot;
    const int32_t* tables; int64_t sbt_n;
    const int32_t* lens;
    void* out; int out_dtype; int64_t so_t, so_n, so_h;
    int T; int64_t n_seqs; int Hq, Hkv, n_rep, passes;
    int bs_log2; int64_t max_blocks, num_blocks;
    float scale;
    float* ws; int splits; int chunk_keys;
    uint32_t* status;
    int64_t items;
};

struct Plan {
    int R;        // query heads served per pass over K/V
    int passes;   // passes per KV head
    int splits;   // key ranges per sequence
    int chunk;    // keys per range (multiple of 32)
    int64_t rec;  // floats per partial record
};

static inline Plan make_plan(int T, int64_t n_seqs, int Hq, int Hkv, int head_dim, int block_size,
                             int64_t max_blocks) {
    Plan p;
    const int n_rep = Hq / Hkv;
    if (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 7 || n_rep == 8) p.R = n_rep;
    else if (n_rep == 3) p.R = 4;
    else if (n_rep < 8) p.R = 8;
    else p.R = (n_rep % 7 == 0) ? 7 : 8;
    p.passes = (n_rep + p.R - 1) / p.R;
    const int64_t max_keys = max_blocks * block_size;
    const int64_t base_items = n_seqs * T * Hkv * p.passes;
    int64_t want = base_items > 0 ? (kTargetWarps + base_items - 1) / base_items : 1;
    if (want < 1) want = 1;
    int64_t chunk = (max_keys + want - 1) / want;
    chunk = ((chunk + 31) / 32) * 32;
    if (chunk < 128) chunk = 128;
    if (chunk > 512) chunk = 512;
    int64_t splits = (max_keys + chunk - 1) / chunk;
    if (splits > kMaxSplits) {
        splits = kMaxSplits;
        chunk = (((max_keys + splits - 1) / splits + 31) / 32) * 32;
        splits = (max_keys + chunk - 1) / chunk;
    }
    if (splits < 1) splits = 1;
    p.splits = static_cast<int>(splits);
    p.chunk = static_cast<int>(chunk);
    p.rec = static_cast<int64_t>(p.R) * (head_dim + 1);
    return p;
}

template <int W>
struct Map {
    static constexpr int KPI = (W == 1) ? 8 : (W == 2) ? 4 : 2;  // keys per phase-B iteration
    static constexpr int LPK = 32 / KPI;                          // lanes per key
    static constexpr int CPL = W * KPI;                           // channels per lane
};

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
    if (dtype == SPK_F32) static_cast<float*>(out)[idx] = v;
    else if (dtype == SPK_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(out)[idx] = __float2half_rn(v);
}

// Loads the W words of one K or V row.  VEC: the row is W-word aligned and may be read with one
// 8- or 16-byte access.
template <int W, bool VEC>
__device__ __forceinline__ void load_row(const uint32_t* p, bool ok, uint32_t (&r)[W]) {
#pragma unroll
    for (int w = 0; w < W; ++w) r[w] = 0;
    if (!ok) return;
    if (VEC && W == 2) {
        const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
        r[0] = t.x; r[1] = t.y;
    } else if (VEC && W == 4) {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
        r[0] = t.x; r[1] = t.y; r[2] = t.z; r[3] = t.w;
    } else {
#pragma unroll
        for (int w = 0; w < W; ++w) r[w] = __ldg(p + w);
    }
}

template <int W, int R, bool VEC>
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const AttnParams p) {
    using M = Map<W>;
    constexpr int D = 32 * W;
    constexpr int LUTN = D + 1;
    __shared__ __align__(16) uint32_t stage_all[kWarpsPerBlock][32][kStageWords];
    __shared__ float lut_all[kWarpsPerBlock][R * LUTN];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
    if (item >= p.items) return;

    // item -> (n, gp, t, c), key range fastest
    int64_t rest = item;
    const int c = static_cast<int>(rest % p.splits); rest /= p.splits;
    const int t = static_cast<int>(rest % p.T); rest /= p.T;
    const int gp = static_cast<int>(rest % (p.Hkv * p.passes)); rest /= (p.Hkv * p.passes);
    const int64_t n = rest;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * R;
    const int nh = min(R, p.n_rep - pass * R);

    int64_t len = p.lens[n];
    const int64_t max_keys = p.max_blocks << p.bs_log2;
    if (len < 1 || len > max_keys) {
        if (lane == 0 && c == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
        len = len < 1 ? 0 : max_keys;
    }
    const int64_t begin = static_cast<int64_t>(c) * p.chunk_keys;
    if (begin >= len && !(len == 0 && c == 0 && p.splits == 1)) return;
    const int64_t end = min(len, begin + p.chunk_keys);

    uint32_t (*stage)[kStageWords] = stage_all[warp];
    float* lut = lut_all[warp];

    // Query words of the heads served here, and their popcounts (the softmax bound).
    uint32_t qw[R][W];
    int cmax[R];
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
        cmax[hh] = 0;
#pragma unroll
        for (int w = 0; w < W; ++w) {
            qw[hh][w] = 0;
            if (hh < nh) qw[hh][w] = __ldg(p.q + t * p.sq_t + n * p.sq_n + (h0 + hh) * p.sq_h + w);
            cmax[hh] += __popc(qw[hh][w]);
        }
    }
    // Weight table: lut[hh][s] = exp((s - cmax[hh]) * scale), s <= cmax[hh].
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
        for (int s = lane; s <= cmax[hh]; s += 32)
            lut[hh * LUTN + s] = expf(static_cast<float>(s - cmax[hh]) * p.scale);
    }
    __syncwarp();

    float acc[R][M::CPL];
    float lsum[R];
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
        lsum[hh] = 0.0f;
#pragma unroll
        for (int i = 0; i < M::CPL; ++i) acc[hh][i] = 0.0f;
    }

    const uint32_t* kbase = p.k + t * p.sk_t + g * p.sk_h;
    const uint32_t* vbase = p.v + t * p.sv_t + g * p.sv_h;
    const int32_t* table = p.tables + n * p.sbt_n;
    const int bs_mask = (1 << p.bs_log2) - 1;
    const int grp = lane / M::LPK;
    const int lsub = lane - grp * M::LPK;

    // Three-stage software pipeline over 32-key tiles: block-table entry of tile i+2, K/V rows of
    // tile i+1, arithmetic of tile i.
    auto table_entry = [&](int64_t key) -> int32_t {
        return key < end ? __ldg(table + (key >> p.bs_log2)) : -1;
    };
    int32_t phys_a = table_entry(begin + lane);        // tile 0
    int32_t phys_b = table_entry(begin + 32 + lane);   // tile 1
    uint32_t kn[W], vn[W];
    bool ok_n;
    {
        const int64_t key = begin + lane;
        ok_n = key < end;
        if (ok_n && (phys_a < 0 || phys_a >= p.num_blocks)) {
            spk_flag(p.status, SPK_STATUS_BAD_BLOCK);
            ok_n = false;
        }
        const int64_t slot = key & bs_mask;
        load_row<W, VEC>(kbase + static_cast<int64_t>(phys_a) * p.sk_blk + slot * p.sk_slot, ok_n, kn);
        load_row<W, VEC>(vbase + static_cast<int64_t>(phys_a) * p.sv_blk + slot * p.sv_slot, ok_n, vn);
    }

    for (int64_t tile = begin; tile < end; tile += 32) {
        uint32_t kc[W], vc[W];
#pragma unroll
        for (int w = 0; w < W; ++w) { kc[w] = kn[w]; vc[w] = vn[w]; }
        const bool ok_c = ok_n;
        // prefetch
        const int32_t phys_c = table_entry(tile + 64 + lane);
        {
            const int64_t key = tile + 32 + lane;
            ok_n = key < end;
            if (ok_n && (phys_b < 0 || phys_b >= p.num_blocks)) {
                spk_flag(p.status, SPK_STATUS_BAD_BLOCK);
                ok_n = false;
            }
            const int64_t slot = key & bs_mask;
            load_row<W, VEC>(kbase + static_cast<int64_t>(phys_b) * p.sk_blk + slot * p.sk_slot, ok_n, kn);
            load_row<W, VEC>(vbase + static_cast<int64_t>(phys_b) * p.sv_blk + slot * p.sv_slot, ok_n, vn);
        }
        phys_b = phys_c;

        // ---- phase A: lane = key ------------------------------------------------
        float wgt[8];
#pragma unroll
        for (int hh = 0; hh < 8; ++hh) wgt[hh] = 0.0f;
#pragma unroll
        for (int hh = 0; hh < R; ++hh) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < W; ++w) s += __popc(qw[hh][w] & kc[w]);
            const float wv = ok_c ? lut[hh * LUTN + s] : 0.0f;
            wgt[hh] = wv;
            lsum[hh] += wv;
        }
        uint4* row = reinterpret_cast<uint4*>(stage[lane]);
        row[0] = make_uint4(__float_as_uint(wgt[0]), __float_as_uint(wgt[1]),
                            __float_as_uint(wgt[2]), __float_as_uint(wgt[3]));
        if (R > 4)
            row[1] = make_uint4(__float_as_uint(wgt[4]), __float_as_uint(wgt[5]),
                                __float_as_uint(wgt[6]), __float_as_uint(wgt[7]));
        {
            uint32_t vv[4] = {0, 0, 0, 0};
#pragma unroll
            for (int w = 0; w < W; ++w) vv[w] = vc[w];
            row[2] = make_uint4(vv[0], vv[1], vv[2], vv[3]);
        }
        __syncwarp();

        // ---- phase B: lane = channel group, KPI keys per iteration -------------------
        const int n_valid = (end - tile) < 32 ? static_cast<int>(end - tile) : 32;
        const int iters = (n_valid + M::KPI - 1) / M::KPI;
#pragma unroll 4
        for (int it = 0; it < iters; ++it) {
            const uint4* r = reinterpret_cast<const uint4*>(stage[it * M::KPI + grp]);
            const uint4 a = r[0];
            uint4 b = make_uint4(0, 0, 0, 0);
            if (R > 4) b = r[1];
            const uint4 vv4 = r[2];
            const float wv[8] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z),
                                 __uint_as_float(a.w), __uint_as_float(b.x), __uint_as_float(b.y),
                                 __uint_as_float(b.z), __uint_as_float(b.w)};
            const uint32_t vv[4] = {vv4.x, vv4.y, vv4.z, vv4.w};
#pragma unroll
            for (int w = 0; w < W; ++w) {
#pragma unroll
                for (int i = 0; i < M::KPI; ++i) {
                    if (vv[w] & (1u << (lsub + M::LPK * i))) {
#pragma unroll
                        for (int hh = 0; hh < R; ++hh) acc[hh][w * M::KPI + i] += wv[hh];
                    }
                }
            }
        }
        __syncwarp();
    }

    // ---- reduce: weights over all lanes, accumulators over the key groups -----------
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) lsum[hh] += __shfl_xor_sync(0xffffffffu, lsum[hh], o);
#pragma unroll
        for (int i = 0; i < M::CPL; ++i) {
#pragma unroll
            for (int o = 16; o >= M::LPK; o >>= 1)
                acc[hh][i] += __shfl_xor_sync(0xffffffffu, acc[hh][i], o);
        }
    }

    if (p.splits == 1) {
#pragma unroll
        for (int hh = 0; hh < R; ++hh) {
            if (hh < nh && (hh % M::KPI) == grp) {
                const int64_t o = t * p.so_t + n * p.so_n + (h0 + hh) * p.so_h;
#pragma unroll
                for (int w = 0; w < W; ++w) {
#pragma unroll
                    for (int i = 0; i < M::KPI; ++i) {
                        const int d = w * 32 + lsub + M::LPK * i;
                        const float val = len > 0 ? acc[hh][w * M::KPI + i] / lsum[hh] : 0.0f;
                        store_out(p.out, p.out_dtype, o + d, val);
                    }
                }
            }
        }
    } else {
        float* rec = p.ws + item * (static_cast<int64_t>(R) * (D + 1));
#pragma unroll
        for (int hh = 0; hh < R; ++hh) {
            if ((hh % M::KPI) == grp) {
#pragma unroll
                for (int w = 0; w < W; ++w) {
#pragma unroll
                    for (int i = 0; i < M::KPI; ++i)
                        rec[hh * D + w * 32 + lsub + M::LPK * i] = acc[hh][w * M::KPI + i];
                }
            }
            if (lane == 0) rec[R * D + hh] = lsum[hh];
        }
    }
}

// Sums the partial records of a (sequence, timestep, KV head, pass) in key-range order and divides.
template <int R>
__global__ void __launch_bounds__(128)
attn_combine_kernel(const AttnParams p, int D) {
    const int64_t grp_item = blockIdx.x;  // (n, gp, t)
    int64_t rest = grp_item;
    const int t = static_cast<int>(rest % p.T); rest /= p.T;
    const int gp = static_cast<int>(rest % (p.Hkv * p.passes)); rest /= (p.Hkv * p.passes);
    const int64_t n = rest;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * R;
    const int nh = min(R, p.n_rep - pass * R);

    int64_t len = p.lens[n];
    const int64_t max_keys = p.max_blocks << p.bs_log2;
    if (len < 1) len = 0;
    if (len > max_keys) len = max_keys;
    const int n_splits = static_cast<int>((len + p.chunk_keys - 1) / p.chunk_keys);
    const int64_t rec_floats = static_cast<int64_t>(R) * (D + 1);
    const float* base = p.ws + grp_item * p.splits * rec_floats;
    for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
        const int hh = idx / D;
        const int d = idx - hh * D;
        float a = 0.0f, l = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            a += base[s * rec_floats + hh * D + d];
            l += base[s * rec_floats + R * D + hh];
        }
        const float val = n_splits > 0 ? a / l : 0.0f;
        store_out(p.out, p.out_dtype, t * p.so_t + n * p.so_n + (h0 + hh) * p.so_h + d, val);
    }
}

template <int W, int R>
int launch_attn(const AttnParams& p, bool vec, cudaStream_t stream) {
    const int64_t blocks = (p.items + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    if (vec && (W == 2 || W == 4))
        attn_decode_kernel<W, R, true><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(p);
    else
        attn_decode_kernel<W, R, false><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(p);
    SPK_CHECK_LAUNCH();
    if (p.splits > 1) {
        const int64_t groups = p.items / p.splits;
        attn_combine_kernel<R><<<static_cast<unsigned>(groups), 128, 0, stream>>>(p, 32 * W);
        SPK_CHECK_LAUNCH();
    }
    return SPK_OK;
}

template <int W>
int dispatch_r(const AttnParams& p, int R, bool vec, cudaStream_t stream) {
    switch (R) {
        case 1: return launch_attn<W, 1>(p, vec, stream);
        case 2: return launch_attn<W, 2>(p, vec, stream);
        case 4: return launch_attn<W, 4>(p, vec, stream);
        case 7: return launch_attn<W, 7>(p, vec, stream);
        case 8: return launch_attn<W, 8>(p, vec, stream);
        default: return SPK_ERR_UNSUPPORTED;
    }
}

static inline int log2_exact(int x) {
    if (x < 1 || (x & (x - 1)) != 0) return -1;
    int l = 0;
    while ((1 << l) < x) ++l;
    return l;
}

static inline bool aligned_to(const void* ptr, int64_t a, int64_t b, int64_t c, int64_t d, int words) {
    const int64_t bytes = static_cast<int64_t>(words) * 4;
    return (reinterpret_cast<uintptr_t>(ptr) % bytes == 0) && (a % words == 0) && (b % words == 0) &&
           (c % words == 0) && (d % words == 0);
}

// ---------------------------------------------------------------------------
// Exact scores, for checking the integer half on its own.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
qk_scores_kernel(const uint32_t* __restrict__ q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                 const uint32_t* __restrict__ k, int64_t sk_t, int64_t sk_h, int64_t sk_blk,
                 int64_t sk_slot, const int32_t* __restrict__ tables, int64_t sbt_n,
                 const int32_t* __restrict__ lens, int32_t* __restrict__ scores, int64_t max_len,
                 int T, int64_t n_seqs, int Hq, int n_rep, int W, int bs_log2, int64_t max_blocks,
                 int64_t num_blocks, uint32_t* status) {
    // grid.x over key tiles, grid.y = (t, n, h) flattened
    int64_t rest = blockIdx.y;
    const int h = static_cast<int>(rest % Hq); rest /= Hq;
    const int64_t n = rest % n_seqs;
    const int t = static_cast<int>(rest / n_seqs);
    const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (j >= max_len) return;
    int64_t len = lens[n];
    const int64_t max_keys = max_blocks << bs_log2;
    if (len < 0) len = 0;
    if (len > max_keys) len = max_keys;
    int32_t s = -1;
    if (j < len) {
        const int32_t phys = tables[n * sbt_n + (j >> bs_log2)];
        if (phys < 0 || phys >= num_blocks) {
            spk_flag(status, SPK_STATUS_BAD_BLOCK);
        } else {
            const uint32_t* kp = k + t * sk_t + (h / n_rep) * sk_h + static_cast<int64_t>(phys) * sk_blk +
                                 (j & ((1 << bs_log2) - 1)) * sk_slot;
            const uint32_t* qp = q + t * sq_t + n * sq_n + h * sq_h;
            s = 0;
            for (int w = 0; w < W; ++w) s += __popc(qp[w] & kp[w]);
        }
    }
    scores[((static_cast<int64_t>(t) * n_seqs + n) * Hq + h) * max_len + j] = s;
}

template <typename TO>
__global__ void __launch_bounds__(256)
gather_unpack_kernel(const uint32_t* __restrict__ cache, int64_t s_t, int64_t s_h, int64_t s_blk,
                     int64_t s_slot, const int32_t* __restrict__ table, int64_t seq_len, int T,
                     int Hkv, int D, int bs_log2, int64_t num_blocks, TO* __restrict__ out,
                     uint32_t* status) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t total = static_cast<int64_t>(T) * Hkv * seq_len * D;
    if (idx >= total) return;
    int64_t rest = idx;
    const int c = static_cast<int>(rest % D); rest /= D;
    const int64_t s = rest % seq_len; rest /= seq_len;
    const int h = static_cast<int>(rest % Hkv);
    const int t = static_cast<int>(rest / Hkv);
    const int32_t phys = table[s >> bs_log2];
    bool bit = false;
    if (phys < 0 || phys >= num_blocks) {
        spk_flag(status, SPK_STATUS_BAD_BLOCK);
    } else {
        const uint32_t word = cache[t * s_t + h * s_h + static_cast<int64_t>(phys) * s_blk +
                                    (s & ((1 << bs_log2) - 1)) * s_slot + (c >> 5)];
        bit = (word >> (c & 31)) & 1u;
    }
    out[idx] = spk_bit_as<TO>(bit);
}

}  // namespace

extern "C" int64_t spk_attn_decode_workspace_bytes(int T, int64_t n_seqs, int num_q_heads,
                                                   int num_kv_heads, int head_dim, int block_size,
                                                   int64_t max_blocks) {
    if (T < 1 || n_seqs < 1 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 32 ||
        head_dim > 128 || head_dim % 32 != 0 || num_q_heads % num_kv_heads != 0 ||
        log2_exact(block_size) < 0 || max_blocks < 1)
        return 0;
    const Plan pl = make_plan(T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks);
    if (pl.splits == 1) return 0;
    return n_seqs * T * num_kv_heads * pl.passes * pl.splits * pl.rec * static_cast<int64_t>(sizeof(float));
}

extern "C" int spk_attn_decode(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                               const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                               const int32_t* v, int64_t sv_t, int64_t sv_h, int64_t sv_blk, int64_t sv_slot,
                               const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                               void* out, int out_dtype, int64_t so_t, int64_t so_n, int64_t so_h,
                               int T, int64_t n_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                               int block_size, int64_t max_blocks, int64_t num_blocks, float scale,
                               void* workspace, int64_t workspace_bytes, uint32_t* status, void* stream) {
    if (T < 0 || n_seqs < 0 || num_q_heads < 1 || num_kv_heads < 1 || max_blocks < 1 || num_blocks < 1)
        return SPK_ERR_BAD_SHAPE;
    if (num_q_heads % num_kv_heads != 0) return SPK_ERR_BAD_SHAPE;
    if (head_dim < 32 || head_dim > 128 || head_dim % 32 != 0) return SPK_ERR_UNSUPPORTED;
    const int bs_log2 = log2_exact(block_size);
    if (bs_log2 < 0) return SPK_ERR_UNSUPPORTED;
    if (out_dtype != SPK_F32 && out_dtype != SPK_BF16 && out_dtype != SPK_F16) return SPK_ERR_BAD_DTYPE;
    if (T == 0 || n_seqs == 0) return SPK_OK;
    if (q == nullptr || k == nullptr || v == nullptr || block_tables == nullptr ||
        seq_lens == nullptr || out == nullptr)
        return SPK_ERR_NULL_POINTER;

    const Plan pl = make_plan(T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks);
    const int64_t need = pl.splits == 1 ? 0
        : n_seqs * T * num_kv_heads * pl.passes * pl.splits * pl.rec * static_cast<int64_t>(sizeof(float));
    if (need > 0 && (workspace == nullptr || workspace_bytes < need)) return SPK_ERR_WORKSPACE_TOO_SMALL;

    AttnParams p;
    p.q = reinterpret_cast<const uint32_t*>(q); p.sq_t = sq_t; p.sq_n = sq_n; p.sq_h = sq_h;
    p.k = reinterpret_cast<const uint32_t*>(k); p.sk_t = sk_t; p.sk_h = sk_h; p.sk_blk = sk_blk; p.sk_slot = sk_slot;
    p.v = reinterpret_cast<const uint32_t*>(v); p.sv_t = sv_t; p.sv_h = sv_h; p.sv_blk = sv_blk; p.sv_slot = sv_slot;
    p.tables = block_tables; p.sbt_n = sbt_n; p.lens = seq_lens;
    p.out = out; p.out_dtype = out_dtype; p.so_t = so_t; p.so_n = so_n; p.so_h = so_h;
    p.T = T; p.n_seqs = n_seqs; p.Hq = num_q_heads; p.Hkv = num_kv_heads;
    p.n_rep = num_q_heads / num_kv_heads; p.passes = pl.passes;
    p.bs_log2 = bs_log2; p.max_blocks = max_blocks; p.num_blocks = num_blocks;
    p.scale = scale; p.ws = static_cast<float*>(workspace); p.splits = pl.splits; p.chunk_keys = pl.chunk;
    p.status = status;
    p.items = n_seqs * T * num_kv_heads * pl.passes * pl.splits;

    const int W = head_dim / 32;
    const bool vec = aligned_to(k, sk_t, sk_h, sk_blk, sk_slot, W) && aligned_to(v, sv_t, sv_h, sv_blk, sv_slot, W);
    cudaStream_t s = spk_stream(stream);
    switch (W) {
        case 1: return dispatch_r<1>(p, pl.R, vec, s);
        case 2: return dispatch_r<2>(p, pl.R, vec, s);
        case 3: return dispatch_r<3>(p, pl.R, vec, s);
        case 4: return dispatch_r<4>(p, pl.R, vec, s);
        default: return SPK_ERR_UNSUPPORTED;
    }
}

extern "C" int spk_qk_scores(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                             const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                             const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                             int32_t* scores, int64_t max_len, int T, int64_t n_seqs, int num_q_heads,
                             int num_kv_heads, int head_dim, int block_size, int64_t max_blocks,
                             int64_t num_blocks, uint32_t* status, void* stream) {
    if (T < 0 || n_seqs < 0 || num_q_heads < 1 || num_kv_heads < 1 || max_blocks < 1 || num_blocks < 1 ||
        max_len < 0 || num_q_heads % num_kv_heads != 0)
        return SPK_ERR_BAD_SHAPE;
    if (head_dim < 32 || head_dim % 32 != 0) return SPK_ERR_UNSUPPORTED;
    const int bs_log2 = log2_exact(block_size);
    if (bs_log2 < 0) return SPK_ERR_UNSUPPORTED;
    if (T == 0 || n_seqs == 0 || max_len == 0) return SPK_OK;
    if (q == nullptr || k == nullptr || block_tables == nullptr || seq_lens == nullptr || scores == nullptr)
        return SPK_ERR_NULL_POINTER;
    const int64_t rows = static_cast<int64_t>(T) * n_seqs * num_q_heads;
    if (rows > 65535) return SPK_ERR_TOO_LARGE;
    dim3 grid(static_cast<unsigned>((max_len + 127) / 128), static_cast<unsigned>(rows));
    qk_scores_kernel<<<grid, 128, 0, spk_stream(stream)>>>(
        reinterpret_cast<const uint32_t*>(q), sq_t, sq_n, sq_h, reinterpret_cast<const uint32_t*>(k),
        sk_t, sk_h, sk_blk, sk_slot, block_tables, sbt_n, seq_lens, scores, max_len, T, n_seqs,
        num_q_heads, num_q_heads / num_kv_heads, head_dim / 32, bs_log2, max_blocks, num_blocks, status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_gather_kv_unpacked(const int32_t* cache, int64_t s_t, int64_t s_h, int64_t s_blk,
                                      int64_t s_slot, const int32_t* block_table, int64_t seq_len,
                                      int T, int num_kv_heads, int head_dim, int block_size,
                                      int64_t num_blocks, void* out, int out_dtype, uint32_t* status,
                                      void* stream) {
    if (T < 0 || num_kv_heads < 1 || head_dim < 1 || seq_len < 0 || num_blocks < 1) return SPK_ERR_BAD_SHAPE;
    const int bs_log2 = log2_exact(block_size);
    if (bs_log2 < 0) return SPK_ERR_UNSUPPORTED;
    if (T == 0 || seq_len == 0) return SPK_OK;
    if (cache == nullptr || block_table == nullptr || out == nullptr) return SPK_ERR_NULL_POINTER;
    const int64_t total = static_cast<int64_t>(T) * num_kv_heads * seq_len * head_dim;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    const unsigned gsz = static_cast<unsigned>(blocks);
    cudaStream_t s = spk_stream(stream);
    const uint32_t* c = reinterpret_cast<const uint32_t*>(cache);
#define SPK_GATHER(TO)                                                                          \
    gather_unpack_kernel<TO><<<gsz, 256, 0, s>>>(c, s_t, s_h, s_blk, s_slot, block_table, seq_len, T, \
                                                 num_kv_heads, head_dim, bs_log2, num_blocks,  \
                                                 static_cast<TO*>(out), status)
    switch (out_dtype) {
        case SPK_F32: SPK_GATHER(float); break;
        case SPK_BF16: SPK_GATHER(__nv_bfloat16); break;
        case SPK_F16: SPK_GATHER(__half); break;
        case SPK_U8: SPK_GATHER(uint8_t); break;
        default: return SPK_ERR_BAD_DTYPE;
    }
#undef SPK_GATHER
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
