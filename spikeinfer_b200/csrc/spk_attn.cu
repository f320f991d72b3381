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

constexpr int kMaxWarps = 4;  // warps per CTA: 4, or 2 for batches of short rows (see make_plan)
constexpr int kMaxSplits = 256;
#ifndef SPK_ATTN_CHUNK_MAX
#define SPK_ATTN_CHUNK_MAX 4096
#endif
#ifndef SPK_ATTN_MIN_BLOCKS
#define SPK_ATTN_MIN_BLOCKS 1
#endif
constexpr int kWaveWarps = 148 * 12;  // warps resident at once (twelve per SM at the kernel's register count)
#ifndef SPK_ATTN_SHORT_ROW_KEYS
#define SPK_ATTN_SHORT_ROW_KEYS 0  // two-warp CTAs measured slower (17.7 us against 12.6 us at 64 rows x 160 keys): off
#endif

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
    float* ws; int splits; int granule;  // granule: keys per CTA step, 32 x warps per CTA
    uint32_t* status;
    int64_t items;
};

struct Plan {
    int R;        // query heads served per pass over K/V
    int passes;   // passes per KV head
    int splits;   // key ranges per sequence
    int chunk;    // keys per range (multiple of the granule)
    int warps;    // warps per CTA
    int64_t rec;  // floats per partial record
};

static inline Plan make_plan(int T, int64_t n_seqs, int Hq, int Hkv, int head_dim, int block_size,
                             int64_t max_blocks) {
    Plan p;
    const int n_rep = Hq / Hkv;
#ifdef SPK_ATTN_SPLIT7
    if (n_rep == 7) p.R = 4; else
#endif
    if (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 7 || n_rep == 8) p.R = n_rep;
    else if (n_rep == 3) p.R = 4;
    else if (n_rep < 8) p.R = 8;
    else p.R = (n_rep % 7 == 0) ? 7 : 8;
    p.passes = (n_rep + p.R - 1) / p.R;
    // One CTA serves one (row, key range); its warps take the range's 32-key tiles round-robin, so a
    // range is a whole number of granules (one tile per warp).  Rows are cut only as far as needed to
    // fill the GPU once, and never into ranges above SPK_ATTN_CHUNK_MAX keys, so that ragged batches
    // balance; when every row fits one range the kernel writes the output itself and no combine
    // launch follows.  Four warps per CTA, except for a batch of short rows that four-warp CTAs would
    // spread over a little more than one resident wave: two-warp CTAs then keep every row resident at
    // once (the kernel is latency bound there, and a second wave doubles its duration).
    const int64_t max_keys = max_blocks * block_size;
    const int64_t base_items = n_seqs * T * Hkv * p.passes;
    p.warps = 4;
    if (max_keys <= SPK_ATTN_SHORT_ROW_KEYS && base_items * 4 > kWaveWarps && base_items * 2 <= kWaveWarps)
        p.warps = 2;
    const int granule = 32 * p.warps;
    const int64_t target = kWaveWarps / p.warps;
    int64_t want = base_items > 0 ? (target + base_items - 1) / base_items : 1;
    if (want < 1) want = 1;
    int64_t chunk = (max_keys + want - 1) / want;
    chunk = ((chunk + granule - 1) / granule) * granule;
    if (chunk > SPK_ATTN_CHUNK_MAX) chunk = SPK_ATTN_CHUNK_MAX;
    int64_t splits = (max_keys + chunk - 1) / chunk;
    if (splits > kMaxSplits) {
        splits = kMaxSplits;
        chunk = (((max_keys + splits - 1) / splits + granule - 1) / granule) * granule;
        splits = (max_keys + chunk - 1) / chunk;
    }
    if (splits < 1) splits = 1;
    p.splits = static_cast<int>(splits);
    p.chunk = static_cast<int>(chunk);
    p.rec = static_cast<int64_t>(p.R) * head_dim + 8;  // R*D sums, then R (padded to 8) weight totals
    return p;
}

template <int W>
struct Map {
    // Phase-B lane mapping: a key is served by LPK lanes, lane `ls` of the group owns the 8 channels
    // of byte `ls` of the V row (word ls / 4, byte ls % 4).  KPI keys are processed per iteration.
    static constexpr int LPK = (W == 1) ? 4 : (W == 2) ? 8 : 16;
    static constexpr int KPI = 32 / LPK;
    static constexpr int ITERS = 32 / KPI;
};

// Staged row of one key: the R weights (padded to a multiple of 4 words), then the V words.  The row
// length is an odd multiple of 4 words so that both the per-key 16-byte stores of phase A and the
// per-group 16-byte broadcast loads of phase B are free of bank conflicts.
template <int W, int R>
struct Row {
    static constexpr int NQ = (R + 3) / 4;  // 16-byte loads that cover the weights
    static constexpr int V_OFF = (R + W <= 4 * NQ) ? R : 4 * NQ;
    static constexpr int NEED = ((V_OFF + W + 3) / 4) * 4;
    static constexpr int WORDS = (NEED / 4) % 2 == 1 ? NEED : NEED + 4;
};

// Weights are kept multiplied by 2^kScaleLog2 so that the products below stay normal numbers.
constexpr int kScaleLog2 = 40;

// Keys per range of a row of `len` keys cut into at most `splits` ranges of whole granules.
__device__ __forceinline__ int64_t row_range_keys(int64_t len, int splits, int granule) {
    const int64_t gr = (len + granule - 1) / granule;
    const int64_t n = gr < splits ? (gr > 0 ? gr : 1) : splits;
    return ((gr + n - 1) / n) * granule;
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
    if (dtype == SPK_F32) static_cast<float*>(out)[idx] = v;
    else if (dtype == SPK_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(out)[idx] = __float2half_rn(v);
}

// Packed pair of fp32 values in one 64-bit register (the operand type of the f32x2 instructions).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// acc = a * b + acc on both halves (one instruction, two fp32 FMAs).
__device__ __forceinline__ void fma2(uint64_t& acc, uint64_t a, uint64_t b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
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

// Phase B of one 32-key tile: every staged key is broadcast to the LPK lanes that serve it; a lane adds
// the key's weights to the accumulators of those of its 8 channels whose V bit is set.
//
// The V byte a lane owns is rotated so that its 8 bits sit at bit positions 23..30 of a register;
// masking one of those bits and reading the result as fp32 gives either 0 or the power of two
// c_i = 2^(2^i - 127).  fma(weight, that, acc) therefore IS the bit-selected add, scaled by c_i; the
// scale is exact (no product leaves the normal range, see kScaleLog2) and is removed once, after the
// last key.  Two channels share one f32x2 FMA.  Measured on B200, this form beats per-bit predicated
// adds (47 us against 68-73 us per call at 64 sequences x [128, 4096] keys) and scalar FMAs on the
// same masks (51 us against 60 us).
typedef uint64_t AccT;    // two channels per f32x2 accumulator
constexpr int kAccPerLane = 4;

template <int W, int R>
__device__ __forceinline__ void phase_b(const uint32_t* stage, int grp, int ls, AccT (&acc)[R][kAccPerLane]) {
    using M = Map<W>;
    using RW = Row<W, R>;
    const int word_off = RW::V_OFF + (ls >> 2);         // V word inside the staged row
    const bool idle = ls >= 4 * W;                      // W == 3: lanes 12..15 own no channels
    const int rot = (23 - 8 * (ls & 3)) & 31;           // rotate-left amount
#pragma unroll  // fully unrolled: partial unrolling (1, 2, 4) measured 6-18 % slower
    for (int it = 0; it < M::ITERS; ++it) {
        const uint32_t* row = stage + (it * M::KPI + grp) * RW::WORDS;
        float w[4 * RW::NQ];
#pragma unroll
        for (int j = 0; j < RW::NQ; ++j) {
            const float4 t = *reinterpret_cast<const float4*>(row + 4 * j);
            w[4 * j] = t.x; w[4 * j + 1] = t.y; w[4 * j + 2] = t.z; w[4 * j + 3] = t.w;
        }
        uint32_t v = idle ? 0u : row[word_off];
        v = __funnelshift_l(v, v, rot);
        uint64_t m[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            m[i] = pack2(__uint_as_float(v & (1u << (23 + 2 * i))), __uint_as_float(v & (1u << (24 + 2 * i))));
#pragma unroll
        for (int hh = 0; hh < R; ++hh) {
            const uint64_t w2 = pack2(w[hh], w[hh]);
#pragma unroll
            for (int i = 0; i < 4; ++i) fma2(acc[hh][i], w2, m[i]);
        }
    }
}

template <int W, int R, bool VEC, int NW>
__global__ void __launch_bounds__(32 * NW, SPK_ATTN_MIN_BLOCKS)
attn_decode_kernel(const AttnParams p) {
    constexpr int kThreads = 32 * NW;
    constexpr int kGranule = 32 * NW;
    using M = Map<W>;
    constexpr int D = 32 * W;
    constexpr int LUTN = D + 1;
    using RW = Row<W, R>;
    constexpr int REC = R * D + 8;  // R*D sums, then the R weight totals (padded to 8)
    __shared__ __align__(16) uint32_t stage_all[NW][32 * RW::WORDS];
    // R weight tables followed by an all-zero copy that lanes past the end of the key range read
    __shared__ float lut[2 * R * LUTN];
    __shared__ __align__(16) float red[NW][REC];  // per-warp partial sums, folded at the end

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // One CTA per item; its warps take the 32-key tiles of the item's key range round-robin.  Every
    // exit below depends on the item only, so the whole CTA leaves together (barriers stay legal).
    const int64_t item = blockIdx.x;

    // item -> (n, c, gp, t): timestep fastest, so neighbouring CTAs walk the same pages
    int64_t rest = item;
    const int t = static_cast<int>(rest % p.T); rest /= p.T;
    const int gp = static_cast<int>(rest % (p.Hkv * p.passes)); rest /= (p.Hkv * p.passes);
    const int c = static_cast<int>(rest % p.splits); rest /= p.splits;
    int64_t n = rest;
    if (p.n_seqs <= 128 && p.n_seqs > 1) {
        // Longest rows first (coarsely): rows are ranked by length class (8 classes of max_keys / 8 keys),
        // ties by index, and this item serves the row of rank `rest`.  The long-running CTAs are thus
        // scheduled early and the last wave holds short rows.  Ballots over the lengths held one or a
        // few per lane: a few dozen instructions per warp.
        const int64_t max_keys_ = p.max_blocks << p.bs_log2;
        int shift = 0;
        while ((max_keys_ >> shift) > 8) ++shift;
        int cls[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int j = lane + 32 * k;
            int v = -1;
            if (j < p.n_seqs) {
                const int lj = p.lens[j];
                v = lj <= 0 ? 0 : min(7, (lj - 1) >> shift);
            }
            cls[k] = v;
        }
        int want = static_cast<int>(rest);
        int found = 0;
        bool done = false;
        for (int c8 = 7; c8 >= 0 && !done; --c8) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const unsigned m = __ballot_sync(0xffffffffu, cls[k] == c8);
                const int cnt = __popc(m);
                if (!done) {
                    if (want < cnt) {
                        found = 32 * k + static_cast<int>(__fns(m, 0, want + 1));
                        done = true;
                    } else {
                        want -= cnt;
                    }
                }
            }
        }
        n = found;
    }
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * R;
    const int nh = min(R, p.n_rep - pass * R);

    int64_t len = p.lens[n];
    const int64_t max_keys = p.max_blocks << p.bs_log2;
    if (len < 1 || len > max_keys) {
        if (threadIdx.x == 0 && c == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
        len = len < 1 ? 0 : max_keys;
    }
    // A row is cut into up to `splits` equal key ranges of whole granules, whatever its length: short
    // rows are spread over several CTAs too (short critical path when the GPU is underfilled).
    const int64_t range = row_range_keys(len, p.splits, p.granule);
    const int64_t begin = static_cast<int64_t>(c) * range;
    if (begin >= len && !(len == 0 && c == 0 && p.splits == 1)) return;
    const int64_t end = min(len, begin + range);

    uint32_t* stage = stage_all[warp];
    const int64_t first = begin + 32 * warp;  // this warp's first tile; the next one is kGranule keys on

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
    AccT acc[R][kAccPerLane];
    float lsum[R];
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
        lsum[hh] = 0.0f;
#pragma unroll
        for (int i = 0; i < kAccPerLane; ++i) acc[hh][i] = 0;
    }

    const uint32_t* kbase = p.k + t * p.sk_t + g * p.sk_h;
    const uint32_t* vbase = p.v + t * p.sv_t + g * p.sv_h;
    const int32_t* table = p.tables + n * p.sbt_n;
    const int bs_mask = (1 << p.bs_log2) - 1;
    const int grp = lane / M::LPK;
    const int ls = lane - grp * M::LPK;

    // Three-stage software pipeline over 32-key tiles: block-table entry of tile i+2, K/V rows of
    // tile i+1, arithmetic of tile i.
    auto table_entry = [&](int64_t key) -> int32_t {
        return key < end ? __ldg(table + (key >> p.bs_log2)) : -1;
    };
    auto fetch = [&](int64_t key, int32_t phys, uint32_t (&kr)[W], uint32_t (&vr)[W]) -> bool {
        bool ok = key < end;
        if (ok && (phys < 0 || phys >= p.num_blocks)) {
            spk_flag(p.status, SPK_STATUS_BAD_BLOCK);
            ok = false;
        }
        const int64_t slot = key & bs_mask;
        load_row<W, VEC>(kbase + static_cast<int64_t>(phys) * p.sk_blk + slot * p.sk_slot, ok, kr);
        load_row<W, VEC>(vbase + static_cast<int64_t>(phys) * p.sv_blk + slot * p.sv_slot, ok, vr);
        return ok;
    };
    int32_t phys_b = table_entry(first + kGranule + lane);  // this warp's second tile
    uint32_t kn[W], vn[W];
    bool ok_n = fetch(first + lane, table_entry(first + lane), kn, vn);

    // (built after the first loads were issued, so their latency overlaps the exponentials)
    // Weight table: lut[hh][s] = 2^kScaleLog2 * exp((s - cmax[hh]) * scale) for s <= cmax[hh]; the
    // second half of the array stays zero.
    for (int i = threadIdx.x; i < R * LUTN; i += kThreads) lut[R * LUTN + i] = 0.0f;
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
        for (int s = threadIdx.x; s <= cmax[hh]; s += kThreads)
            lut[hh * LUTN + s] = ldexpf(expf(static_cast<float>(s - cmax[hh]) * p.scale), kScaleLog2);
    }
    __syncthreads();

    for (int64_t tile = first; tile < end; tile += kGranule) {
        uint32_t kc[W], vc[W];
#pragma unroll
        for (int w = 0; w < W; ++w) { kc[w] = kn[w]; vc[w] = vn[w]; }
        const bool ok_c = ok_n;
        const int32_t phys_c = table_entry(tile + 2 * kGranule + lane);
        ok_n = fetch(tile + kGranule + lane, phys_b, kn, vn);
        phys_b = phys_c;

        // ---- phase A: lane = key ------------------------------------------------
        const float* my_lut = lut + (ok_c ? 0 : R * LUTN);
        uint32_t rowv[RW::WORDS];
#pragma unroll
        for (int i = 0; i < RW::WORDS; ++i) rowv[i] = 0u;
#pragma unroll
        for (int hh = 0; hh < R; ++hh) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < W; ++w) s += __popc(qw[hh][w] & kc[w]);
            const float wv = my_lut[hh * LUTN + s];
            rowv[hh] = __float_as_uint(wv);
            lsum[hh] += wv;
        }
#pragma unroll
        for (int w = 0; w < W; ++w) rowv[RW::V_OFF + w] = vc[w];
        uint4* row = reinterpret_cast<uint4*>(stage + lane * RW::WORDS);
#pragma unroll
        for (int j = 0; j < RW::NEED / 4; ++j)
            row[j] = make_uint4(rowv[4 * j], rowv[4 * j + 1], rowv[4 * j + 2], rowv[4 * j + 3]);
        __syncwarp();
        // ---- phase B: lane = (key group, V byte) ---------------------------------
        phase_b<W, R>(stage, grp, ls, acc);
        __syncwarp();
    }

    // ---- reduce: weights over all lanes, accumulators over the key groups; undo the scales ---
    float out_v[R][8];
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) lsum[hh] += __shfl_xor_sync(0xffffffffu, lsum[hh], o);
#pragma unroll
        for (int i = 0; i < 4; ++i) unpack2(acc[hh][i], out_v[hh][2 * i], out_v[hh][2 * i + 1]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int o = 16; o >= M::LPK; o >>= 1) out_v[hh][i] += __shfl_xor_sync(0xffffffffu, out_v[hh][i], o);
            // channel i carries the factor 2^(2^i - 127)
            out_v[hh][i] *= __uint_as_float((254u - (1u << i)) << 23);
        }
    }
    // out_v and lsum both carry the common factor 2^kScaleLog2.  Fold the four warps through shared
    // memory; the CTA then writes either the output row (the row has one range) or one partial record.
    const int d0 = (ls >> 2) * 32 + (ls & 3) * 8;
    const bool owner = ls < 4 * W;
#pragma unroll
    for (int hh = 0; hh < R; ++hh) {
        if (owner && (hh % M::KPI) == grp) {
            float4* o = reinterpret_cast<float4*>(&red[warp][hh * D + d0]);
            o[0] = make_float4(out_v[hh][0], out_v[hh][1], out_v[hh][2], out_v[hh][3]);
            o[1] = make_float4(out_v[hh][4], out_v[hh][5], out_v[hh][6], out_v[hh][7]);
        }
        if (lane == 0) red[warp][R * D + hh] = lsum[hh];
    }
    if (lane >= R && lane < 8) red[warp][R * D + lane] = 0.0f;
    __syncthreads();
    if (p.splits == 1) {
        for (int idx = threadIdx.x; idx < nh * D; idx += kThreads) {
            const int hh = idx / D;
            const int d = idx - hh * D;
            float a = 0.0f, l = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) { a += red[w][idx]; l += red[w][R * D + hh]; }
            store_out(p.out, p.out_dtype, t * p.so_t + n * p.so_n + (h0 + hh) * p.so_h + d,
                      len > 0 ? a / l : 0.0f);
        }
    } else {
        const int64_t rec_idx = ((n * (p.Hkv * p.passes) + gp) * p.T + t) * p.splits + c;
        float* rec = p.ws + rec_idx * REC;
        for (int idx = threadIdx.x; idx < REC; idx += kThreads) {
            float a = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; ++w) a += red[w][idx];
            rec[idx] = a;
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
    const int64_t range = row_range_keys(len, p.splits, p.granule);
    const int n_splits = static_cast<int>((len + range - 1) / range);
    const int64_t rec_floats = static_cast<int64_t>(R) * D + 8;
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

template <int W, int R, int NW>
int launch_attn_nw(const AttnParams& p, bool vec, cudaStream_t stream) {
    const int64_t blocks = p.items;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    if (vec && (W == 2 || W == 4))
        attn_decode_kernel<W, R, true, NW><<<static_cast<unsigned>(blocks), 32 * NW, 0, stream>>>(p);
    else
        attn_decode_kernel<W, R, false, NW><<<static_cast<unsigned>(blocks), 32 * NW, 0, stream>>>(p);
    SPK_CHECK_LAUNCH();
    if (p.splits > 1) {
        const int64_t groups = p.items / p.splits;
        attn_combine_kernel<R><<<static_cast<unsigned>(groups), 128, 0, stream>>>(p, 32 * W);
        SPK_CHECK_LAUNCH();
    }
    return SPK_OK;
}

template <int W, int R>
int launch_attn(const AttnParams& p, bool vec, cudaStream_t stream) {
    return p.granule == 64 ? launch_attn_nw<W, R, 2>(p, vec, stream) : launch_attn_nw<W, R, 4>(p, vec, stream);
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
    p.scale = scale; p.ws = static_cast<float*>(workspace); p.splits = pl.splits; p.granule = 32 * pl.warps;
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

// ---------------------------------------------------------------------------
// Allocation-free variant of spk_attn_decode.
//
// Some callers have no way to provide the split-KV workspace: a serving process that gave every
// remaining byte of HBM to the page pool when it started (a later cudaMalloc can fail, and it
// synchronises the device), or a host that reaches this library through a thin FFI and only ever
// holds the device pointers it was handed.  For them the partial sums go to a fixed array that is
// part of the loaded module, so each GPU that loads the library carries these 8 MiB until the
// process exits, whether or not the entry point is ever called.
// ---------------------------------------------------------------------------
constexpr int64_t kStaticScratchBytes = SPK_ATTN_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) float g_attn_static_scratch[kStaticScratchBytes / sizeof(float)];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_ptr[kMaxDevices] = {};  // per device, filled on first use

// Device address of the array on the current device.  The array's name is only a host-side handle:
// the address a kernel can use has to be asked for, once per device, with that device current.
static int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return spk_set_cuda_error(e);
    if (dev < 0 || dev >= kMaxDevices) return SPK_ERR_UNSUPPORTED;
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess) return spk_set_cuda_error(e);
        g_static_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_static_scratch_ptr[dev];
    return SPK_OK;
}

extern "C" int64_t spk_attn_decode_static_capacity(void) { return kStaticScratchBytes; }

extern "C" int spk_attn_decode_static(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                                      const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                                      const int32_t* v, int64_t sv_t, int64_t sv_h, int64_t sv_blk, int64_t sv_slot,
                                      const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                                      void* out, int out_dtype, int64_t so_t, int64_t so_n, int64_t so_h,
                                      int T, int64_t n_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                      int block_size, int64_t max_blocks, int64_t num_blocks, float scale,
                                      uint32_t* status, void* stream) {
    const int64_t need = spk_attn_decode_workspace_bytes(T, n_seqs, num_q_heads, num_kv_heads, head_dim,
                                                         block_size, max_blocks);
    if (need > kStaticScratchBytes) return SPK_ERR_STATIC_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    if (need > 0) {
        const int rc = static_scratch_for_current_device(&scratch);
        if (rc != SPK_OK) return rc;
    }
    // Every partial record the combine pass reads is written earlier in the same call, so the
    // array needs no clearing between calls; whatever the previous call left is never read.
    return spk_attn_decode(q, sq_t, sq_n, sq_h, k, sk_t, sk_h, sk_blk, sk_slot, v, sv_t, sv_h, sv_blk, sv_slot,
                           block_tables, sbt_n, seq_lens, out, out_dtype, so_t, so_n, so_h, T, n_seqs,
                           num_q_heads, num_kv_heads, head_dim, block_size, max_blocks, num_blocks, scale,
                           scratch, need, status, stream);
}
