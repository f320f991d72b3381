// Paged popcount decode attention over bit-packed spike K/V.
//
// out[t,n,h,:] = softmax_j( popc(q[t,n,h] & k_j) * scale ) . v_j   over the keys of sequence n
// (spikeinfer/kernels/spike_attention.py:67-150 of the reference).
//
// Formulation used here:
//  * A CTA owns one work item = (sequence, timestep, KV head, key range) and serves all query heads
//    of the GQA group (eight per pass) from a single read of K and V; its warps take the range's
//    32-key tiles round-robin and fold their partial sums through shared memory at the end.
//  * popc(q & k) <= popc(q), so the softmax is taken against the fixed bound m = popc(q)*scale
//    instead of a running maximum.  That is the same softmax (a common factor cancels) and it cannot
//    overflow.  Partial sums of different key ranges therefore combine by plain addition.
//  * A score is an integer in [0, popc(q)], so a weight takes at most head_dim+1 values: they come
//    from a per-item table in shared memory, indexed by the exact integer score.
//  * The weighted sum over keys is a small matrix product, heads x keys times keys x channels, with a
//    0/1 right-hand side.  It runs on the tensor cores as m16n8k16 fp16 MMAs with fp32 accumulation:
//      - left operand: the weight of (head, key), split into two fp16 numbers hi + lo * 2^-11 that
//        occupy rows h and h + 8 of the 16-row tile (22 significant bits together; the table holds
//        the pair ready-made);
//      - right operand: the V bit of (key, channel) used IN PLACE as an fp16 number.  The V rows of two
//        consecutive keys are staged interleaved by half-word and all bits but one are masked off; what is
//        left is either 0 or the fp16 subnormal 2^(i-24) for bit i.  Products with it are exact, and
//        the known power of two is removed from the accumulators once, after the last key;
//    The softmax denominators are plain fp32 sums of the same weights (a second table lookup per key).
//    One 32-key tile of a 64-channel head costs 16 MMAs and about 220 instructions per warp, against
//    about 620 instructions for the same tile as fp32 bit-selected adds on the SIMT pipes.  No single
//    unit is the limit (halving the MMAs as a timing probe, dropping a third of the integer operations,
//    a quarter of the shared-memory traffic or doubling the resident warps each moved the time by
//    -3 % .. +20 %); the kernel is bound by dependency latency within a warp's tile.
#include "spk_attn.cuh"

#include <atomic>

namespace {

constexpr int kHeads = kAttnHeads;    // query heads per pass: rows 0..7 (hi) and 8..15 (lo) of the MMA tile
constexpr int kMaxSplits = 256;
#ifndef SPK_ATTN_CHUNK_MAX
#define SPK_ATTN_CHUNK_MAX 4096
#endif
#ifndef SPK_ATTN_WIDE_CTA_KEYS
#define SPK_ATTN_WIDE_CTA_KEYS 2048
#endif
#ifndef SPK_ATTN_SM_WARPS
#define SPK_ATTN_SM_WARPS 16
#endif
constexpr int kSmWarps = SPK_ATTN_SM_WARPS;  // resident warps per SM: the kernel is held to 128 registers
// Weights are kept multiplied by 2^kScaleLog2: the largest (score = bound) is 2^14, inside the fp16
// range, and the fp16 pair stays accurate down to exp(-24) of it.
constexpr int kScaleLog2 = 14;
constexpr float kMaxExponentRange = 24.0f;  // head_dim * scale above this is refused
constexpr int kLutStride = 2 * 129 + 6;       // words between the fp16-pair tables and their fp32 twins
constexpr float kLoUnscale = 1.0f / 2048.0f;  // the lo half of a weight is stored times 2^11

struct Plan {
    int passes;   // passes per KV head (eight query heads each)
    int warps;    // warps per CTA: 4, or 8 for a single wave of long rows
    int splits;   // key ranges per sequence
    int chunk;    // keys per range (multiple of the granule)
    int64_t rec;  // floats per partial record
};

// A range is a whole number of granules (one 32-key tile per warp of the CTA).  Rows are cut only as far
// as needed to fill the GPU once, and never into ranges above SPK_ATTN_CHUNK_MAX keys; when every row
// fits one range the kernel writes the output itself and no combine launch follows.
static inline void plan_ranges(Plan& p, int64_t base_items, int64_t max_keys) {
    const int granule = 32 * p.warps;
    const int64_t target = 148 * (kSmWarps / p.warps);
    int64_t want = base_items > 0 ? target / base_items : 1;  // cut only while that still fits one wave
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
}

static inline Plan make_plan(int T, int64_t n_seqs, int Hq, int Hkv, int head_dim, int block_size,
                             int64_t max_blocks) {
    Plan p;
    const int n_rep = Hq / Hkv;
    p.passes = (n_rep + kHeads - 1) / kHeads;
    const int64_t max_keys = max_blocks * block_size;
    const int64_t base_items = n_seqs * T * Hkv * p.passes;
    p.warps = 4;
    plan_ranges(p, base_items, max_keys);
    // Long rows whose CTAs are all resident at once: the longest row sets the duration, so give every
    // row eight warps (measured at 64 ragged rows of up to 4096 keys: 24.6 us against 26.7 us).
    // (head_dim 128: the eight partial-sum buffers would not fit the static shared memory)
    if (head_dim <= 96 && max_keys >= SPK_ATTN_WIDE_CTA_KEYS && base_items * p.splits <= 148 * (kSmWarps / 4)) {
        p.warps = 8;
        plan_ranges(p, base_items, max_keys);
    }
    p.rec = static_cast<int64_t>(kHeads) * head_dim + 8;  // 8*D sums, then the 8 weight totals
    return p;
}

// Keys per range of a row of `len` keys cut into at most `splits` ranges of whole granules.
__device__ __forceinline__ int row_range_keys(int len, int splits, int granule) {
    const int gr = (len + granule - 1) / granule;
    const int n = gr < splits ? (gr > 0 ? gr : 1) : splits;
    return ((gr + n - 1) / n) * granule;
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t idx, float v) {
    if (dtype == SPK_F32) static_cast<float*>(out)[idx] = v;
    else if (dtype == SPK_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(out)[idx] = __float2half_rn(v);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// c += a (16x16 fp16, row major) * b (16x8 fp16, column major), fp32 accumulators.  Thread (gid =
// lane / 4, tig = lane % 4) holds a0 = A[gid][2tig..], a1 = A[gid+8][2tig..], a2 = A[gid][2tig+8..],
// a3 = A[gid+8][2tig+8..]; b0 = B[2tig..][gid], b1 = B[2tig+8..][gid]; c0,c1 = C[gid][2tig, 2tig+1],
// c2,c3 = C[gid+8][2tig, 2tig+1] (two consecutive elements per register, lower index in the low half).
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Loads the W words of one K or V row.  VEC: the row is W-word aligned and may be read with one
// 8- or 16-byte access.
template <int W, bool VEC>
__device__ __forceinline__ void load_row(const uint32_t* p, bool ok, uint32_t (&r)[W]) {
    // (selects, not branches: the address is always a valid one, dead keys read slot 0 of page 0)
    if (VEC && W == 2) {
        const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
        r[0] = ok ? t.x : 0u; r[1] = ok ? t.y : 0u;
    } else if (VEC && W == 4) {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
        r[0] = ok ? t.x : 0u; r[1] = ok ? t.y : 0u; r[2] = ok ? t.z : 0u; r[3] = ok ? t.w : 0u;
    } else {
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const uint32_t t = __ldg(p + w);
            r[w] = ok ? t : 0u;
        }
    }
}

// Stores one staged row (W words, W-word aligned) with a single access where the width allows.
template <int W>
__device__ __forceinline__ void store_row(uint32_t* p, const uint32_t (&r)[W]) {
    if (W == 2) *reinterpret_cast<uint2*>(p) = make_uint2(r[0], r[1]);
    else if (W == 4) *reinterpret_cast<uint4*>(p) = make_uint4(r[0], r[1], r[2], r[3]);
    else {
#pragma unroll
        for (int w = 0; w < W; ++w) p[w] = r[w];
    }
}

// N consecutive staged words, 4N-byte aligned when N is a power of two and 8-byte aligned otherwise
// (the rows of a key pair).
template <int N>
__device__ __forceinline__ void load_words(const uint32_t* p, uint32_t (&r)[N]) {
    if (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const uint4 t = reinterpret_cast<const uint4*>(p)[i];
            r[4 * i] = t.x; r[4 * i + 1] = t.y; r[4 * i + 2] = t.z; r[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            const uint2 t = reinterpret_cast<const uint2*>(p)[i];
            r[2 * i] = t.x; r[2 * i + 1] = t.y;
        }
    }
}

// V bits as fp16 numbers.  The V rows of a key pair (k, k + 1) are staged interleaved by half-word:
// word h of the pair holds bits 16h..16h+15 of key k in its low half and of key k + 1 in its high half,
// which is the register layout of the MMA's right operand (two consecutive keys, one channel).  Masking
// one bit per half leaves 0 or a power of two:
//   bits 0..9 are fp16 mantissa bits: 2^(b-24) (subnormal); bits 10..14 exponent bits: 2^(2^(b-10) - 15);
//   bit 15 is the sign and unusable, so the threads of column 7 (gid 7) read a second copy of the staging
//   in which every half-word is shifted right by one, and mask bits 6 and 14 instead of 7 and 15.
// The power of two depends only on (column, byte parity) and is removed from the accumulators at the end.
struct VBits {
    __device__ static __forceinline__ int bit(int col, int odd_byte) {
        return col == 7 ? (odd_byte ? 14 : 6) : col + 8 * odd_byte;
    }
    __device__ static __forceinline__ uint32_t mask(int col, int odd_byte) {
        const uint32_t b = 1u << bit(col, odd_byte);
        return b | (b << 16);
    }
    // log2 of the fp16 value of that single bit
    __device__ static __forceinline__ int log2_value(int col, int odd_byte) {
        const int b = bit(col, odd_byte);
        return b < 10 ? b - 24 : (1 << (b - 10)) - 15;
    }
};

// One 32-key tile of a warp, from the staged K and V rows.  ALL: every key of the tile is live
// (`live` is all ones); otherwise keys whose bit in `live` is clear get weight zero.
//
// The MMAs accumulate in place over all tiles of the warp.  Against an fp64 evaluation the result is off
// by 6.0e-7 (relative to the largest output) after 32768 keys; starting every MMA from zero and adding
// its result with an ordinary fp32 add gave the same figure, so the in-place form loses nothing.
template <int W, bool ALL>
__device__ __forceinline__ void tile_mma(const uint32_t* kst, const uint32_t* vst, const uint32_t (&qw)[W],
                                         const uint32_t* my_lut, const uint32_t* zero_lut, unsigned live,
                                         int gid, int tig, float (&acc)[4 * W][4], float& lsum) {
    // Bit kept from each half-word for the even / odd byte of a half-word (see VBits below).
    const uint32_t m0 = VBits::mask(gid, 0), m1 = VBits::mask(gid, 1);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        // this thread's keys of the 16-key step: k0, k0 + 1, k0 + 8, k0 + 9
        const int k0 = 16 * ks + 2 * tig;
        uint32_t kw[2][2 * W], vx[2][2 * W];  // [key pair][words]: K rows of the two keys; interleaved V
        load_words<2 * W>(kst + k0 * W, kw[0]);
        load_words<2 * W>(kst + (k0 + 8) * W, kw[1]);
        load_words<2 * W>(vst + k0 * W, vx[0]);
        load_words<2 * W>(vst + (k0 + 8) * W, vx[1]);
        // weights of (head gid, these keys): {hi, lo} fp16 pairs from the table, indexed by bound - score
        uint32_t wt[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < W; ++w) s += __popc(qw[w] & kw[i >> 1][(i & 1) * W + w]);
            const int key = k0 + (i & 1) + 8 * (i >> 1);
            const uint32_t* tab = (ALL || ((live >> key) & 1u)) ? my_lut : zero_lut;
            wt[i] = tab[-s];
            lsum += __uint_as_float(tab[kLutStride - s]);  // the same weight in fp32, for the denominator
        }
        uint32_t a[4];
        a[0] = prmt(wt[0], wt[1], 0x5410);  // hi(k0), hi(k0+1)      -> row gid
        a[1] = prmt(wt[0], wt[1], 0x7632);  // lo(k0), lo(k0+1)      -> row gid + 8
        a[2] = prmt(wt[2], wt[3], 0x5410);  // hi(k0+8), hi(k0+9)
        a[3] = prmt(wt[2], wt[3], 0x7632);
        // V bits of channel 8j + gid for the same keys, as fp16: half-word pair j / 2 of each key pair,
        // all bits but this thread's one masked off.
#pragma unroll
        for (int j = 0; j < 4 * W; ++j) {
            const uint32_t m = (j & 1) ? m1 : m0;
            mma16816(acc[j], a, vx[0][j >> 1] & m, vx[1][j >> 1] & m);
        }
    }
}

template <int W, bool VEC, int NW>
__global__ void __launch_bounds__(32 * NW, kSmWarps / NW)
attn_decode_kernel(const AttnParams p) {
    constexpr int kWarps = NW;
    constexpr int kThreads = 32 * NW;
    constexpr int kGranule = 32 * NW;  // keys per CTA step
    constexpr int D = 32 * W;
    constexpr int LUTN = D + 1;
    constexpr int REC = kHeads * D + 8;  // 8*D sums, then the 8 weight totals
    __shared__ __align__(16) uint32_t kst_all[kWarps][32 * W];
    __shared__ __align__(16) uint32_t vst_all[kWarps][2][32 * W];  // interleaved V pairs; [1] = shifted copy
    // weight tables indexed by bound - score: {hi, lo} fp16 pairs, then (kLutStride words on) the same
    // weights in fp32; an all-zero copy of both for dead keys and absent heads sits LUTN words further
    static_assert(2 * LUTN <= kLutStride, "table stride");
    __shared__ uint32_t lut[2 * kLutStride];
    // per-warp partial sums, folded at the end; head rows padded by 8 floats against bank conflicts
    constexpr int RS = D + 8;
    __shared__ __align__(16) float red[kWarps][kHeads * RS + 8];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int gid = lane >> 2;  // MMA row group: the query head this thread weighs keys for
    const int tig = lane & 3;
    // One CTA per item; every exit below depends on the item only, so the whole CTA leaves together.
    const int64_t item = blockIdx.x;

    // item -> (n, c, gp, t): timestep fastest, so neighbouring CTAs walk the same pages
    int64_t rest = item;
    const int t = static_cast<int>(rest % p.T); rest /= p.T;
    const int gp = static_cast<int>(rest % (p.Hkv * p.passes)); rest /= (p.Hkv * p.passes);
    const int c = static_cast<int>(rest % p.splits); rest /= p.splits;
    int64_t n = rest;
    if (p.longest_first) {
        // Longest rows first (coarsely): rows are ranked by length class (8 classes of max_keys / 8 keys),
        // ties by index, and this item serves the row of rank `rest`.  The long-running CTAs are thus
        // scheduled early and the last wave holds short rows.  Ballots over the lengths held one or a
        // few per lane: a few dozen instructions per warp.
        int shift = 0;
        while ((p.max_keys >> shift) > 8) ++shift;
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
    const int h0 = g * p.n_rep + pass * kHeads;
    const int nh = min(kHeads, p.n_rep - pass * kHeads);

    int len = p.lens[n];
    if (len < 1 || len > p.max_keys) {
        if (threadIdx.x == 0 && c == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
        len = len < 1 ? 0 : p.max_keys;
    }
    // A row is cut into up to `splits` equal key ranges of whole granules, whatever its length: short
    // rows are spread over several CTAs too (short critical path when the GPU is underfilled).
    const int range = row_range_keys(len, p.splits, p.granule);
    const int begin = c * range;
    if (begin >= len && !(len == 0 && c == 0 && p.splits == 1)) return;
    const int end = min(len, begin + range);

    uint32_t* kst = kst_all[warp];
    uint32_t* vst_w = vst_all[warp][0];                              // written at staging time
    const uint32_t* vst = vst_all[warp][gid == 7 ? 1 : 0];           // read as the MMA operand
    const int first = begin + 32 * warp;  // this warp's first tile; the next one is kGranule keys on

    // Query words of this thread's head and their popcount (the softmax bound).
    uint32_t qw[W];
    int cmax = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) {
        qw[w] = gid < nh ? __ldg(p.q + t * p.sq_t + n * p.sq_n + (h0 + gid) * p.sq_h + w) : 0u;
        cmax += __popc(qw[w]);
    }
    float acc[4 * W][4], lsum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4 * W; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    const uint32_t* kbase = p.k + t * p.sk_t + g * p.sk_h;
    const uint32_t* vbase = p.v + t * p.sv_t + g * p.sv_h;
    const int32_t* table = p.tables + n * p.sbt_n;
    const int bs_mask = (1 << p.bs_log2) - 1;

    // Three-stage software pipeline over this warp's tiles: block-table entry of the tile after next,
    // K/V rows of the next tile (lane = key, coalesced), arithmetic of the current one.
    auto table_entry = [&](int key) -> int32_t {
        return key < end ? __ldg(table + (key >> p.bs_log2)) : -1;
    };
    auto fetch = [&](int key, int32_t phys, uint32_t (&kr)[W], uint32_t (&vr)[W]) -> bool {
        const bool in_range = key < end;
        const bool ok = in_range && static_cast<uint32_t>(phys) < static_cast<uint32_t>(p.num_blocks);
        if (in_range && !ok) spk_flag(p.status, SPK_STATUS_BAD_BLOCK);
        const int page = ok ? phys : 0;
        const int slot = ok ? (key & bs_mask) : 0;
        load_row<W, VEC>(kbase + static_cast<int64_t>(page) * p.sk_blk + slot * p.sk_slot, ok, kr);
        load_row<W, VEC>(vbase + static_cast<int64_t>(page) * p.sv_blk + slot * p.sv_slot, ok, vr);
        return ok;
    };
    int32_t phys_b = table_entry(first + kGranule + lane);  // this warp's second tile
    uint32_t kn[W], vn[W];
    bool ok_n = fetch(first + lane, table_entry(first + lane), kn, vn);

    // (built after the first loads were issued, so their latency overlaps the exponentials)
    // A weight depends on bound - score only: lut[d] = {hi, lo} with hi + lo * 2^-11 =
    // 2^kScaleLog2 * exp(-d * scale), d = 0..head_dim, shared by all heads.
    for (int i = threadIdx.x; i < 2 * LUTN; i += kThreads) {
        uint32_t e = 0u, f = 0u;
        if (i < LUTN) {
            const float wv = ldexpf(expf(-static_cast<float>(i) * p.scale), kScaleLog2);
            const __half hi = __float2half_rn(wv);
            const __half lo = __float2half_rn((wv - __half2float(hi)) * 2048.0f);
            e = static_cast<uint32_t>(__half_as_ushort(hi)) | (static_cast<uint32_t>(__half_as_ushort(lo)) << 16);
            f = __float_as_uint(wv);
        }
        lut[i] = e;
        lut[kLutStride + i] = f;
    }
    __syncthreads();
    // tables are indexed with -score from these bases: live keys of a present head read lut[cmax - s],
    // everything else reads a zero (cmax <= head_dim keeps both inside their table)
    const uint32_t* zero_lut = lut + LUTN + cmax;
    const uint32_t* my_lut = gid < nh ? lut + cmax : zero_lut;

    for (int tile = first; tile < end; tile += kGranule) {
        // ---- stage the current tile (lane = key) and start the next one's loads --------------------
        store_row<W>(kst + lane * W, kn);
        {
            // even lanes build the low half-words of their key pair, odd lanes the high ones
            const uint32_t sel = (lane & 1) ? 0x3276u : 0x5410u;
            uint32_t* dst = vst_w + (lane >> 1) * 2 * W + (lane & 1);
#pragma unroll
            for (int w = 0; w < W; ++w) {
                const uint32_t other = __shfl_xor_sync(0xffffffffu, vn[w], 1);
                const uint32_t x = prmt(vn[w], other, sel);
                dst[2 * w] = x;
                dst[32 * W + 2 * w] = (x >> 1) & 0x7fff7fffu;
            }
        }
        const unsigned live = __ballot_sync(0xffffffffu, ok_n);
        const int32_t phys_c = table_entry(tile + 2 * kGranule + lane);
        ok_n = fetch(tile + kGranule + lane, phys_b, kn, vn);
        phys_b = phys_c;
        __syncwarp();
        // ---- weights and weighted sums on the tensor cores (lane = (head, key quad)) -----------------
        if (live == 0xffffffffu) tile_mma<W, true>(kst, vst, qw, my_lut, zero_lut, live, gid, tig, acc, lsum);
        else tile_mma<W, false>(kst, vst, qw, my_lut, zero_lut, live, gid, tig, acc, lsum);
        __syncwarp();
    }

    // ---- undo the scales; fold the warps; write the output row or one partial record --------------
    // A column of a channel block was multiplied by the power of two its V bit reads as (VBits); the lo rows by
    // 2^11.  Sums and totals both keep the common factor 2^kScaleLog2.
    float un[2][2];  // [byte parity][column 2tig, 2tig + 1]: 2^-log2_value
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int i = 0; i < 2; ++i)
            un[e][i] = __uint_as_float(static_cast<uint32_t>(127 - VBits::log2_value(2 * tig + i, e)) << 23);
#pragma unroll
    for (int j = 0; j < 4 * W; ++j) {
        const float v0 = (acc[j][0] + acc[j][2] * kLoUnscale) * un[j & 1][0];
        const float v1 = (acc[j][1] + acc[j][3] * kLoUnscale) * un[j & 1][1];
        *reinterpret_cast<float2*>(&red[warp][gid * RS + 8 * j + 2 * tig]) = make_float2(v0, v1);
    }
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);  // the four threads of a head hold disjoint keys
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
    if (tig == 0) red[warp][kHeads * RS + gid] = lsum;
    __syncthreads();
    if (p.splits == 1) {
        for (int idx = threadIdx.x; idx < nh * D; idx += kThreads) {
            const int hh = idx / D;
            const int d = idx - hh * D;
            float a = 0.0f, l = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) { a += red[w][hh * RS + d]; l += red[w][kHeads * RS + hh]; }
            store_out(p.out, p.out_dtype, t * p.so_t + n * p.so_n + (h0 + hh) * p.so_h + d,
                      len > 0 ? a / l : 0.0f);
        }
    } else {
        const int64_t rec_idx = ((n * (p.Hkv * p.passes) + gp) * p.T + t) * p.splits + c;
        float* rec = p.ws + rec_idx * REC;
        for (int idx = threadIdx.x; idx < REC; idx += kThreads) {
            const int hh = idx / D;  // 8: the weight totals
            const int src = hh * RS + (idx - hh * D);
            float a = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) a += red[w][src];
            rec[idx] = a;
        }
    }
}

// Sums the partial records of a (sequence, timestep, KV head, pass) in key-range order and divides.
__global__ void __launch_bounds__(128)
attn_combine_kernel(const AttnParams p, int D) {
    const int64_t grp_item = blockIdx.x;  // (n, gp, t)
    int64_t rest = grp_item;
    const int t = static_cast<int>(rest % p.T); rest /= p.T;
    const int gp = static_cast<int>(rest % (p.Hkv * p.passes)); rest /= (p.Hkv * p.passes);
    const int64_t n = rest;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * kHeads;
    const int nh = min(kHeads, p.n_rep - pass * kHeads);

    int len = p.lens[n];
    if (len < 1) len = 0;
    if (len > p.max_keys) len = p.max_keys;
    const int range = row_range_keys(len, p.splits, p.granule);
    const int n_splits = (len > 0 && range > 0) ? (len + range - 1) / range : 0;  // an empty row has no records
    const int64_t rec_floats = static_cast<int64_t>(kHeads) * D + 8;
    const float* base = p.ws + grp_item * p.splits * rec_floats;
    for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
        const int hh = idx / D;
        const int d = idx - hh * D;
        float a = 0.0f, l = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            a += base[s * rec_floats + hh * D + d];
            l += base[s * rec_floats + kHeads * D + hh];
        }
        const float val = n_splits > 0 ? a / l : 0.0f;
        store_out(p.out, p.out_dtype, t * p.so_t + n * p.so_n + (h0 + hh) * p.so_h + d, val);
    }
}

template <int W, int NW>
int launch_attn_nw(const AttnParams& p, bool vec, cudaStream_t stream) {
    const int64_t blocks = p.items;
    if (blocks > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    if (vec && (W == 2 || W == 4))
        attn_decode_kernel<W, true, NW><<<static_cast<unsigned>(blocks), 32 * NW, 0, stream>>>(p);
    else
        attn_decode_kernel<W, false, NW><<<static_cast<unsigned>(blocks), 32 * NW, 0, stream>>>(p);
    SPK_CHECK_LAUNCH();
    if (p.splits > 1) {
        const int64_t groups = p.items / p.splits;
        attn_combine_kernel<<<static_cast<unsigned>(groups), 128, 0, stream>>>(p, 32 * W);
        SPK_CHECK_LAUNCH();
    }
    return SPK_OK;
}

template <int W>
int launch_attn(const AttnParams& p, bool vec, cudaStream_t stream) {
    if (W <= 3 && p.granule == 256) return launch_attn_nw<W, (W <= 3 ? 8 : 4)>(p, vec, stream);
    if (p.granule != 128) return SPK_ERR_UNSUPPORTED;
    return launch_attn_nw<W, 4>(p, vec, stream);
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
                     int64_t s_slot, const int32_t* __restrict__ table, int64_t sbt_n, int64_t seq_len, int T,
                     int Hkv, int D, int bs_log2, int64_t num_blocks, TO* __restrict__ out,
                     uint32_t* status) {
    // grid.y = sequence: its row of the block tables, its [T, H_kv, seq_len, D] slab of the output
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t total = static_cast<int64_t>(T) * Hkv * seq_len * D;
    if (idx >= total) return;
    table += blockIdx.y * sbt_n;
    out += blockIdx.y * total;
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

namespace {
thread_local bool g_overlap_next_call = false;
}

extern "C" int spk_attn_overlap_next_call(void) {
    g_overlap_next_call = true;
    return SPK_OK;
}

extern "C" int64_t spk_attn_decode_workspace_bytes(int T, int64_t n_seqs, int num_q_heads,
                                                   int num_kv_heads, int head_dim, int block_size,
                                                   int64_t max_blocks) {
    if (T < 1 || n_seqs < 1 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 32 ||
        head_dim > 128 || head_dim % 32 != 0 || num_q_heads % num_kv_heads != 0 ||
        log2_exact(block_size) < 0 || max_blocks < 1 ||
        max_blocks > (0x7fffffffLL - 3 * 256 - 32) / block_size)  // spk_attn_decode refuses these
        return 0;
    // enough for whichever form of the kernel the call takes
    const Plan pl = make_plan(T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks);
    const int64_t general = pl.splits == 1 ? 0
        : n_seqs * T * num_kv_heads * pl.passes * pl.splits * pl.rec * static_cast<int64_t>(sizeof(float));
    const StreamPlan spl = spk_attn_stream_plan(T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks);
    const int64_t streaming = spl.ok ? spl.ws_bytes : 0;
    return general > streaming ? general : streaming;
}

extern "C" int spk_attn_decode(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                               const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                               const int32_t* v, int64_t sv_t, int64_t sv_h, int64_t sv_blk, int64_t sv_slot,
                               const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                               void* out, int out_dtype, int64_t so_t, int64_t so_n, int64_t so_h,
                               int T, int64_t n_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                               int block_size, int64_t max_blocks, int64_t num_blocks, float scale,
                               void* workspace, int64_t workspace_bytes, uint32_t* status, void* stream) {
    SpkRange nvtx_range("spk_attn_decode");
    const bool overlap = g_overlap_next_call;  // one-shot, consumed whatever happens below
    g_overlap_next_call = false;
    if (T < 0 || n_seqs < 0 || num_q_heads < 1 || num_kv_heads < 1 || max_blocks < 1 || num_blocks < 1)
        return SPK_ERR_BAD_SHAPE;
    if (num_q_heads % num_kv_heads != 0) return SPK_ERR_BAD_SHAPE;
    if (head_dim < 32 || head_dim > 128 || head_dim % 32 != 0) return SPK_ERR_UNSUPPORTED;
    const int bs_log2 = log2_exact(block_size);
    if (bs_log2 < 0) return SPK_ERR_UNSUPPORTED;
    if (out_dtype != SPK_F32 && out_dtype != SPK_BF16 && out_dtype != SPK_F16) return SPK_ERR_BAD_DTYPE;
    // the fp16 weight pairs cover exp(-24)..1 of the bound; head_dim^-0.5 (the reference's scale) gives <= 11.4
    if (!(scale >= 0.0f) || scale * static_cast<float>(head_dim) > kMaxExponentRange) return SPK_ERR_UNSUPPORTED;
    if (T == 0 || n_seqs == 0) return SPK_OK;
    if (q == nullptr || k == nullptr || v == nullptr || block_tables == nullptr ||
        seq_lens == nullptr || out == nullptr)
        return SPK_ERR_NULL_POINTER;

    // the kernel indexes keys, pages and the page/slot strides with 32-bit integers; it forms key indices up to
    // two CTA steps and a tile past a row's end (prefetch), so the largest row stays that far below 2^31
    const int64_t lim = 0x7fffffffLL;
    if ((max_blocks << bs_log2) > lim - 3 * 256 - 32 || max_blocks > lim || num_blocks > lim) return SPK_ERR_TOO_LARGE;
    for (int64_t st : {sk_blk, sk_slot, sv_blk, sv_slot})
        if (st > lim || st < -lim) return SPK_ERR_TOO_LARGE;

    const Plan pl = make_plan(T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks);
    const int64_t need = pl.splits == 1 ? 0
        : n_seqs * T * num_kv_heads * pl.passes * pl.splits * pl.rec * static_cast<int64_t>(sizeof(float));

    AttnParams p;
    p.q = reinterpret_cast<const uint32_t*>(q); p.sq_t = sq_t; p.sq_n = sq_n; p.sq_h = sq_h;
    p.k = reinterpret_cast<const uint32_t*>(k); p.sk_t = sk_t; p.sk_h = sk_h; p.sk_blk = static_cast<int>(sk_blk); p.sk_slot = static_cast<int>(sk_slot);
    p.v = reinterpret_cast<const uint32_t*>(v); p.sv_t = sv_t; p.sv_h = sv_h; p.sv_blk = static_cast<int>(sv_blk); p.sv_slot = static_cast<int>(sv_slot);
    p.tables = block_tables; p.sbt_n = sbt_n; p.lens = seq_lens;
    p.out = out; p.out_dtype = out_dtype; p.so_t = so_t; p.so_n = so_n; p.so_h = so_h;
    p.T = T; p.n_seqs = n_seqs; p.Hq = num_q_heads; p.Hkv = num_kv_heads;
    p.n_rep = num_q_heads / num_kv_heads; p.passes = pl.passes;
    p.bs_log2 = bs_log2; p.max_keys = static_cast<int>(max_blocks << bs_log2); p.num_blocks = static_cast<int>(num_blocks);
    p.scale = scale; p.ws = static_cast<float*>(workspace); p.splits = pl.splits; p.granule = 32 * pl.warps;
    p.status = status;
    p.overlap = overlap ? 1 : 0;
    p.items = n_seqs * T * num_kv_heads * pl.passes * pl.splits;
    // all CTAs resident at once: their order does not matter, and skipping the ranking takes one dependent
    // global load off the start of every CTA
    p.longest_first = n_seqs > 1 && n_seqs <= 128 && p.items > 148LL * (kSmWarps / pl.warps);

    cudaStream_t s = spk_stream(stream);
    // Pages of contiguous, 16-byte aligned rows at head_dim 64 / 128 take the streaming form.
    const StreamPlan spl = spk_attn_stream_plan(T, n_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks);
    if (spl.ok && spk_attn_selected_form() != SPK_ATTN_FORM_GENERAL && spk_attn_stream_layout_ok(p, head_dim)) {
        if (spl.ws_bytes > 0 && (workspace == nullptr || workspace_bytes < spl.ws_bytes)) return SPK_ERR_WORKSPACE_TOO_SMALL;
        p.passes = spl.passes;
        return spk_attn_stream_launch(p, spl, head_dim, s);
    }
    if (need > 0 && (workspace == nullptr || workspace_bytes < need)) return SPK_ERR_WORKSPACE_TOO_SMALL;

    const int W = head_dim / 32;
    const bool vec = aligned_to(k, sk_t, sk_h, sk_blk, sk_slot, W) && aligned_to(v, sv_t, sv_h, sv_blk, sv_slot, W);
    switch (W) {
        case 1: return launch_attn<1>(p, vec, s);
        case 2: return launch_attn<2>(p, vec, s);
        case 3: return launch_attn<3>(p, vec, s);
        case 4: return launch_attn<4>(p, vec, s);
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

extern "C" int spk_gather_kv_unpacked_batch(const int32_t* cache, int64_t s_t, int64_t s_h, int64_t s_blk,
                                            int64_t s_slot, const int32_t* block_tables, int64_t sbt_n,
                                            int64_t n_seqs, int64_t seq_len, int T, int num_kv_heads, int head_dim,
                                            int block_size, int64_t num_blocks, void* out, int out_dtype,
                                            uint32_t* status, void* stream) {
    if (T < 0 || num_kv_heads < 1 || head_dim < 1 || seq_len < 0 || num_blocks < 1 || n_seqs < 0) return SPK_ERR_BAD_SHAPE;
    const int bs_log2 = log2_exact(block_size);
    if (bs_log2 < 0) return SPK_ERR_UNSUPPORTED;
    if (T == 0 || seq_len == 0 || n_seqs == 0) return SPK_OK;
    if (cache == nullptr || block_tables == nullptr || out == nullptr) return SPK_ERR_NULL_POINTER;
    const int64_t total = static_cast<int64_t>(T) * num_kv_heads * seq_len * head_dim;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL || n_seqs > 65535) return SPK_ERR_TOO_LARGE;
    const dim3 gsz(static_cast<unsigned>(blocks), static_cast<unsigned>(n_seqs));
    cudaStream_t s = spk_stream(stream);
    const uint32_t* c = reinterpret_cast<const uint32_t*>(cache);
#define SPK_GATHER(TO)                                                                          \
    gather_unpack_kernel<TO><<<gsz, 256, 0, s>>>(c, s_t, s_h, s_blk, s_slot, block_tables, sbt_n, seq_len, T, \
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

extern "C" int spk_gather_kv_unpacked(const int32_t* cache, int64_t s_t, int64_t s_h, int64_t s_blk,
                                      int64_t s_slot, const int32_t* block_table, int64_t seq_len,
                                      int T, int num_kv_heads, int head_dim, int block_size,
                                      int64_t num_blocks, void* out, int out_dtype, uint32_t* status,
                                      void* stream) {
    return spk_gather_kv_unpacked_batch(cache, s_t, s_h, s_blk, s_slot, block_table, 0, 1, seq_len, T, num_kv_heads,
                                        head_dim, block_size, num_blocks, out, out_dtype, status, stream);
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
// per device, filled on first use; atomic because any host thread may make that first call (two threads
// racing store the same value)
static std::atomic<float*> g_static_scratch_ptr[kMaxDevices];

// Device address of the array on the current device.  The array's name is only a host-side handle:
// the address a kernel can use has to be asked for, once per device, with that device current.
static int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return spk_set_cuda_error(e);
    if (dev < 0 || dev >= kMaxDevices) return SPK_ERR_UNSUPPORTED;
    float* known = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (known == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess) return spk_set_cuda_error(e);
        known = static_cast<float*>(p);
        g_static_scratch_ptr[dev].store(known, std::memory_order_release);
    }
    *out = known;
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
    SpkRange nvtx_range("spk_attn_decode_static");
    const int64_t need = spk_attn_decode_workspace_bytes(T, n_seqs, num_q_heads, num_kv_heads, head_dim,
                                                         block_size, max_blocks);
    if (need > kStaticScratchBytes) return SPK_ERR_STATIC_SCRATCH_TOO_SMALL;
    // The address is looked up on the first call per device whatever the problem needs, so that a small
    // warm-up call at start-up settles it and no later call (possibly inside a stream capture) has to.
    float* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != SPK_OK) return rc;
    // Every partial record the combine pass reads is written earlier in the same call, so the
    // array needs no clearing between calls; whatever the previous call left is never read.
    return spk_attn_decode(q, sq_t, sq_n, sq_h, k, sk_t, sk_h, sk_blk, sk_slot, v, sv_t, sv_h, sv_blk, sv_slot,
                           block_tables, sbt_n, seq_lens, out, out_dtype, so_t, so_n, so_h, T, n_seqs,
                           num_q_heads, num_kv_heads, head_dim, block_size, max_blocks, num_blocks, scale,
                           scratch, need, status, stream);
}
