// Paged popcount decode attention, streaming form (the one the decode engine's layouts take).
//
// out[t,n,h,:] = softmax_j( popc(q[t,n,h] & k_j) * scale ) . v_j   over the keys of sequence n
// (spikeinfer/kernels/spike_attention.py:67-150 of the reference).
//
// Shape of the computation:
//  * Every sequence is cut into units of 512 / 1024 / 2048 keys.  A WARP owns one (unit, KV head, pass,
//    timestep) and runs on its own: no barrier after set-up, no cross-warp fold.  Units are enumerated
//    densely (a prefix sum of the rows' unit counts, built once per CTA in shared memory), so every CTA
//    holds four equally sized pieces of work whatever the mix of row lengths.
//  * K and V pages go from global to shared memory with 16-byte cp.async copies, four 32-key tiles in
//    flight per warp; the unit's block-table entries are staged once.  No register staging, no selects.
//  * Scores: popc(q & k) per (head, key) on the integer pipes, thread = (head, key quad).  A score is an
//    integer in [0, popc(q)], so the softmax weight exp((s - popc(q)) * scale) comes from one table shared by
//    all heads, and partial sums of different units combine by plain addition.
//  * Weighted sum on the tensor cores, transposed: out^T[channel][head] += V^T[channel][key] * P^T[key][head]
//    as mma.sync.m16n8k16 (fp16 in, fp32 accumulate).  Sixteen channels fill the sixteen rows, eight heads
//    the eight columns: nothing of the tile is padding.  The left operand is the V bits IN PLACE: the rows
//    of a key pair are interleaved by half-word once per tile (so that a register holds the same sixteen
//    channels of two consecutive keys) and one lop3 per operand register masks all bits but one; what is left is
//    0 or a power of two (an fp16 subnormal for bits 0..9, a normal for bits 10..14).  Bit 15 is the sign: it is
//    kept together with a forced bit 14, which reads as +2 or -2, and the channel's sum is recovered from
//    the weight total.  The known powers of two are removed once, after the last key.
//  * The weight totals (softmax denominators) come from one more MMA per 16 keys whose left operand is all ones.
//  * 16-bit outputs use one fp16 weight (2^-11 relative, the same rounded weight in numerator and denominator);
//    fp32 output uses a {hi, lo} fp16 pair (22 bits) as a second block of columns.
// Per 32-key tile at head_dim 64: 16 popc, 10 MMAs and about 130 instructions per warp; the integer pipe that
// executes popc (a quarter-rate unit) and the issue slots are the two limits.
#include "spk_attn.cuh"

#include <atomic>

namespace {

constexpr int kWarps = 4;          // independent workers per CTA
constexpr int kThreads = 32 * kWarps;
constexpr int kTileKeys = 64;      // keys per pipeline stage: two 32-key MMA tiles
constexpr int kTblMax = 128;       // block-table entries staged per unit (2048 keys of 16-key pages)
constexpr int kDenseRows = 1024;   // up to this many sequences the units are enumerated densely
constexpr int kScaleLog2 = 14;     // weights are kept times 2^14: the largest is 2^14, the smallest used 2^14 e^-24
constexpr float kLoUnscale = 1.0f / 2048.0f;  // the lo half of a weight is stored times 2^11
constexpr int kResidentWarpsTarget = 148 * 20;  // unit form: units are made smaller until the call has twice this many

constexpr int kXGroup = 32 * 4 + 16;  // words between two groups of four byte-words in the regrouped V tile (padded: bank spread)

struct StreamParams {
    int short_steps;  // range form: an item of at most this many 32-key steps is never cut between warps
    int unit_log2;    // log2 of the keys per unit (unit form)
    int max_units;    // units of the longest possible row (unit form)
    int gt;           // T * Hkv * passes: items per sequence
    int dense;        // up to kDenseRows sequences: equal step ranges per warp; otherwise one warp per unit
    int out_vec;      // output rows may be written with 16-byte stores
    int64_t rec;      // floats per partial record
    int64_t workers;  // warps that share the step list (range form)
    float* dense_ws;  // two record slots per worker (range form)
};

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

// 16 bytes global -> shared, bypassing L1; bytes = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// N consecutive words of shared memory, 16-byte aligned (N = 4 or 8).
template <int N>
__device__ __forceinline__ void load_words(const uint32_t* p, uint32_t (&r)[N]) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        const uint4 t = reinterpret_cast<const uint4*>(p)[i];
        r[4 * i] = t.x; r[4 * i + 1] = t.y; r[4 * i + 2] = t.z; r[4 * i + 3] = t.w;
    }
}

__device__ __forceinline__ int units_of(int len, int unit_log2) {
    const int u = (len + (1 << unit_log2) - 1) >> unit_log2;
    return u > 1 ? u : 1;  // an empty row still has one unit: the one that writes its zeros
}

__device__ __forceinline__ int clamp_len(int len, int max_keys) {
    return len < 1 ? 0 : (len > max_keys ? max_keys : len);
}

// 32 keys.  kst: their K rows [key][W]; xb: their V rows regrouped by key pair and BYTE: word g of pair p holds
// byte g of key 2p's row in bits 0..7 and byte g of key 2p+1's row in bits 16..23 (the other two bytes are
// don't-care) and sits at xb[(g / 4) * kXGroup + 4 p + g % 4].  Thread gid supplies the channels of byte gid (and, at head_dim 128, of byte
// gid + 8): in channel block j its two rows are bits 2j and 2j+1 of that byte, so one word per key pair feeds
// all blocks, and a masked bit is always an fp16 subnormal 2^(e - 24), e = 0..7.
// rlut: the weight table positioned so that rlut[score] is this head's weight.
// ALL: every key is live; otherwise keys at or beyond `nlive` get weight zero.
template <int W, int NB, bool ALL>
__device__ __forceinline__ void tile_compute(const uint32_t* kst, const uint32_t* xb, const uint32_t (&qw)[W],
                                             const uint32_t* rlut, int nlive, const uint32_t (&ones)[4], int gid,
                                             int tig, float (&acc)[NB][2 * W + 1][4]) {
    constexpr int MB = 2 * W;  // blocks of 16 channels
    const uint32_t* xt = xb + (gid >> 2) * kXGroup + (gid & 3);  // this thread's byte of pair 0
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        // weights of (this thread's head, keys kp, kp+1) for the two key pairs of the 16-key step
        uint32_t bh[2], bl[2];
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            const int kp = 16 * ks + 8 * pr + 2 * tig;
            uint32_t kw[2 * W];
            load_words<2 * W>(kst + kp * W, kw);
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int w = 0; w < W; ++w) {
                s0 += __popc(qw[w] & kw[w]);
                s1 += __popc(qw[w] & kw[W + w]);
            }
            uint32_t e0 = rlut[s0], e1 = rlut[s1];
            if (!ALL) {
                if (kp >= nlive) e0 = 0u;
                if (kp + 1 >= nlive) e1 = 0u;
            }
            bh[pr] = prmt(e0, e1, 0x5410);
            if (NB == 2) bl[pr] = prmt(e0, e1, 0x7632);
        }
#pragma unroll
        for (int hb = 0; hb < W / 2; ++hb) {  // byte gid (and byte gid + 8 at head_dim 128)
            const uint32_t xa = xt[2 * hb * kXGroup + (8 * ks + tig) * 4];
            const uint32_t xc = xt[2 * hb * kXGroup + (8 * ks + 4 + tig) * 4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t m0 = 0x00010001u << (2 * j), m1 = 0x00010001u << (2 * j + 1);
                const uint32_t a[4] = {xa & m0, xa & m1, xc & m0, xc & m1};
                mma16816(acc[0][4 * hb + j], a, bh[0], bh[1]);
                if (NB == 2) mma16816(acc[NB - 1][4 * hb + j], a, bl[0], bl[1]);
            }
        }
        mma16816(acc[0][MB], ones, bh[0], bh[1]);
        if (NB == 2) mma16816(acc[NB - 1][MB], ones, bl[0], bl[1]);
    }
}

template <typename TO>
__device__ __forceinline__ TO to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }

// Writes COUNT consecutive channels of one head from shared memory (fp32, times inv) in the output type.
template <int COUNT, typename TO>
__device__ __forceinline__ void store_channels(TO* dst, const float* src, float inv, bool vec) {
    if (vec) {
        constexpr int PER = 16 / sizeof(TO);  // elements per 16-byte store
#pragma unroll
        for (int c = 0; c < COUNT; c += PER) {
            union { uint4 u; TO e[PER]; } pk;
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const float4 f = *reinterpret_cast<const float4*>(src + c + i);
                pk.e[i] = to_out<TO>(f.x * inv); pk.e[i + 1] = to_out<TO>(f.y * inv);
                pk.e[i + 2] = to_out<TO>(f.z * inv); pk.e[i + 3] = to_out<TO>(f.w * inv);
            }
            *reinterpret_cast<uint4*>(dst + c) = pk.u;
        }
    } else {
        for (int c = 0; c < COUNT; ++c) dst[c] = to_out<TO>(src[c] * inv);
    }
}

#ifndef SPK_STREAM_MINB
#define SPK_STREAM_MINB 4
#endif

#ifndef SPK_STREAM_MINB4
#define SPK_STREAM_MINB4 3
#endif

#ifndef SPK_SHORT_STEPS
#define SPK_SHORT_STEPS 8
#endif
constexpr int kShortSteps = SPK_SHORT_STEPS;  // an item of at most this many 32-key steps (256 keys) is never cut between warps
constexpr int kUncutSteps = 24;  // tables of at most this many steps (768 keys): nothing is cut at all.  One warp walks such
                                 // a row in under 5 us, about what the combine pass adds to a call once anything may be cut

template <int W>
struct StreamSmem {
    static constexpr int D = 32 * W;
#ifndef SPK_STREAM_STAGES2
#define SPK_STREAM_STAGES2 4
#endif
    static constexpr int STAGES = W == 2 ? SPK_STREAM_STAGES2 : 3;  // 64-key tiles in flight per warp
    static constexpr int HALF_WORDS = kTileKeys * W;     // words of a tile's K rows (and of its V rows)
    static constexpr int TILE_WORDS = 2 * HALF_WORDS;    // K rows then V rows
    static constexpr int ES = D + 4;                     // row stride of the epilogue's transposition buffer
    static_assert(STAGES * TILE_WORDS >= kAttnHeads * ES + 8, "the epilogue reuses the warp's ring");
};

// One piece of one (sequence, KV head, pass, timestep): keys [key0, kend) of `row`, on this warp alone.
// `whole`: the piece is the whole sequence, so the output row is written; otherwise a partial record goes to `rec`.
template <int W, int NB>
__device__ __forceinline__ void stream_piece(const AttnParams& p, const StreamParams& sp, int row, int gt, int key0,
                                             int kend, bool whole, float* rec, uint32_t* ring, uint32_t* xb,
                                             int32_t* tbl, const uint32_t* rlut, int lane) {
    using S = StreamSmem<W>;
    constexpr int D = S::D, MB = 2 * W, STAGES = S::STAGES, HALF_WORDS = S::HALF_WORDS, TILE_WORDS = S::TILE_WORDS;
    constexpr int TILE_BYTES = TILE_WORDS * 4, ES = S::ES;
    const int gid = lane >> 2;  // MMA column = query head; MMA rows gid and gid + 8 = channels
    const int tig = lane & 3;
    const int t = gt % p.T;
    const int gp = gt / p.T;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * kAttnHeads;
    const int nh = min(kAttnHeads, p.n_rep - pass * kAttnHeads);

    const int bs_mask = (1 << p.bs_log2) - 1;
    const int span = kTblMax << p.bs_log2;  // keys whose block-table entries fit the staging
    // block-table entries of the stretch [c0, c1) into this warp's staging
    auto stage_tables = [&](int c0, int c1) {
        const int page0 = c0 >> p.bs_log2;
        const int last_page = ((c1 - 1) >> p.bs_log2) - page0;
        const int32_t* table = p.tables + row * p.sbt_n + page0;
        for (int i = lane; i <= last_page; i += 32) {
            int32_t ph = __ldg(table + i);
            if (static_cast<uint32_t>(ph) >= static_cast<uint32_t>(p.num_blocks)) {
                spk_flag(p.status, SPK_STATUS_BAD_BLOCK);
                ph = 0;
            }
            tbl[i] = ph;
        }
    };
    // query words of this thread's head and their popcount (the softmax bound)
    uint32_t qw[W];
    auto load_q = [&]() {
#pragma unroll
        for (int w = 0; w < W; ++w)
            qw[w] = gid < nh ? __ldg(p.q + t * p.sq_t + row * p.sq_n + (h0 + gid) * p.sq_h + w) : 0u;
    };
    if (!p.overlap) load_q();  // in flight together with the table entries
    __syncwarp();  // every lane is done with the previous piece's entries
    stage_tables(key0, min(kend, key0 + span));
    if (p.overlap) {
        // Everything above read lengths and block tables only.  q and the newest K/V rows come from the kernel
        // launched just before this one, which this launch overlaps (programmatic dependent launch): wait for it.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        load_q();
    }
    int cmax = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) cmax += __popc(qw[w]);
    const uint32_t* my_rlut = rlut + (D - cmax);
    uint32_t ones[4];  // fp16 {1, 1}: the left operand of the weight totals (kept in registers, opaque to the compiler)
#pragma unroll
    for (int i = 0; i < 4; ++i) asm volatile("mov.b32 %0, 0x3C003C00;" : "=r"(ones[i]));
    float acc[NB][MB + 1][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int jb = 0; jb <= MB; ++jb) acc[b][jb][0] = acc[b][jb][1] = acc[b][jb][2] = acc[b][jb][3] = 0.0f;

    const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + lane * 16;
    const uint32_t* kbase = p.k + t * p.sk_t + g * p.sk_h;
    const uint32_t* vbase = p.v + t * p.sv_t + g * p.sv_h;

    // the piece in stretches of at most `span` keys: block-table entries staged once per stretch
    for (int c0 = key0; c0 < kend; c0 += span) {
        const int c1 = min(kend, c0 + span);
        const int nkeys = c1 - c0;
        const int ntiles = (nkeys + kTileKeys - 1) / kTileKeys;
        const int page0 = c0 >> p.bs_log2;
        const int last_page = ((c1 - 1) >> p.bs_log2) - page0;
        if (c0 != key0) {
            __syncwarp();  // every lane is done with the previous stretch's entries and ring
            stage_tables(c0, c1);
        }
        __syncwarp();
        // copies: W = 2: lane l moves keys 2l, 2l+1 of the 64-key tile (16 bytes of K, 16 of V);
        // W = 4: keys l and l + 32 (two K and two V segments)
        int issue_key = c0 + (W == 2 ? 2 * lane : lane);
        uint32_t issue_stage = 0;
        auto issue = [&]() {
#pragma unroll
            for (int c = 0; c < (W == 2 ? 1 : 2); ++c) {
                const int key = issue_key + 32 * c;
                const int bytes = key < c1 ? 16 : 0;
                const int pl = min((key >> p.bs_log2) - page0, last_page);  // dead keys: any valid page
                const int off = tbl[pl] * p.sk_blk + (key & bs_mask) * W;   // same page stride for K and V (host-checked)
                const uint32_t dst = ring_addr + issue_stage + c * 512;
                cp_async16(dst, kbase + off, bytes);
                cp_async16(dst + HALF_WORDS * 4, vbase + off, bytes);
            }
            issue_key += kTileKeys;
            issue_stage = issue_stage == (STAGES - 1) * TILE_BYTES ? 0u : issue_stage + TILE_BYTES;
        };
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < ntiles) issue();
            cp_async_commit();
        }
        const uint32_t* kst = ring;
        int nlive = nkeys;
        for (int tile = 0; tile < ntiles; ++tile) {
            cp_async_wait<STAGES - 2>();  // this tile has landed (the newer STAGES - 2 groups may be in flight)
            __syncwarp();                 // ... for every lane; and every lane is done with the previous tile
            if (tile + STAGES - 1 < ntiles) issue();  // into the stage the previous tile occupied
            cp_async_commit();
            // regroup the V rows of every key pair by byte: lane = pair
            {
                const uint32_t* vst = kst + HALF_WORDS + lane * 2 * W;
                uint32_t r[2 * W], x[4 * W];
                load_words<2 * W>(vst, r);  // key 2l: words 0..W-1; key 2l+1: words W..2W-1
#pragma unroll
                for (int gq = 0; gq < 4 * W; ++gq) {
                    // byte gq % 4 of word gq / 4: of key 2l into byte 0, of key 2l+1 into byte 2
                    const uint32_t sel = (gq % 4) * 0x0011u + (4 + gq % 4) * 0x1100u;
                    x[gq] = prmt(r[gq / 4], r[W + gq / 4], sel);
                }
                // the pair's 4W words are stored as W groups of four; group q of all pairs sits X_GROUP words
                // after group q - 1 (a lane's 16-byte stores are then consecutive, and the readers' banks distinct)
#pragma unroll
                for (int q = 0; q < W; ++q)
                    *reinterpret_cast<uint4*>(xb + q * kXGroup + lane * 4) = make_uint4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
            }
            __syncwarp();
            if (nlive >= kTileKeys) {
                tile_compute<W, NB, true>(kst, xb, qw, my_rlut, 32, ones, gid, tig, acc);
                tile_compute<W, NB, true>(kst + 32 * W, xb + 64, qw, my_rlut, 32, ones, gid, tig, acc);
            } else {
                tile_compute<W, NB, false>(kst, xb, qw, my_rlut, nlive, ones, gid, tig, acc);
                if (nlive > 32)
                    tile_compute<W, NB, false>(kst + 32 * W, xb + 64, qw, my_rlut, nlive - 32, ones, gid, tig, acc);
            }
            nlive -= kTileKeys;
            kst = (tile % STAGES == STAGES - 1) ? ring : kst + TILE_WORDS;
        }
        cp_async_wait<0>();
    }
    __syncwarp();  // the ring is free: the epilogue transposes through it

    // ---- undo the scales, transpose through shared memory, write the output row or a partial record -------
    // In channel block j of byte b (b = gid, or gid + 8 for the second half at head_dim 128) row gid is channel
    // 8b + 2j and row gid + 8 is channel 8b + 2j + 1; a masked bit e read as the fp16 subnormal 2^(e - 24).
    float* ep = reinterpret_cast<float*>(ring);
    float tot0 = acc[0][MB][0], tot1 = acc[0][MB][1];  // weight totals of heads 2tig and 2tig + 1
    if (NB == 2) {
        tot0 += acc[NB - 1][MB][0] * kLoUnscale;
        tot1 += acc[NB - 1][MB][1] * kLoUnscale;
    }
#pragma unroll
    for (int jb = 0; jb < MB; ++jb) {
        float c0 = acc[0][jb][0], c1 = acc[0][jb][1], c2 = acc[0][jb][2], c3 = acc[0][jb][3];
        if (NB == 2) {
            c0 += acc[NB - 1][jb][0] * kLoUnscale; c1 += acc[NB - 1][jb][1] * kLoUnscale;
            c2 += acc[NB - 1][jb][2] * kLoUnscale; c3 += acc[NB - 1][jb][3] * kLoUnscale;
        }
        const int e = 2 * (jb & 3);
        const float f0 = __uint_as_float(static_cast<uint32_t>(127 + 24 - e) << 23);
        const float f1 = __uint_as_float(static_cast<uint32_t>(127 + 23 - e) << 23);
        const int ch = 8 * (gid + 8 * (jb >> 2)) + e;
        *reinterpret_cast<float2*>(ep + (2 * tig) * ES + ch) = make_float2(c0 * f0, c2 * f1);
        *reinterpret_cast<float2*>(ep + (2 * tig + 1) * ES + ch) = make_float2(c1 * f0, c3 * f1);
    }
    if (gid == 0) {
        ep[kAttnHeads * ES + 2 * tig] = tot0;
        ep[kAttnHeads * ES + 2 * tig + 1] = tot1;
    }
    __syncwarp();
    // lane -> (head, quarter of the channels)
    const int hh = lane >> 2;
    constexpr int QC = D / 4;
    const float* src = ep + hh * ES + tig * QC;
    if (whole) {
        if (hh < nh) {
            const float tot = ep[kAttnHeads * ES + hh];
            const float inv = tot > 0.0f ? 1.0f / tot : 0.0f;
            const int64_t idx = t * p.so_t + row * p.so_n + (h0 + hh) * p.so_h + tig * QC;
            if (p.out_dtype == SPK_F32) store_channels<QC>(static_cast<float*>(p.out) + idx, src, inv, sp.out_vec);
            else if (p.out_dtype == SPK_BF16) store_channels<QC>(static_cast<__nv_bfloat16*>(p.out) + idx, src, inv, sp.out_vec);
            else store_channels<QC>(static_cast<__half*>(p.out) + idx, src, inv, sp.out_vec);
        }
    } else {
        store_channels<QC>(rec + hh * D + tig * QC, src, 1.0f, true);
        if (lane < kAttnHeads) rec[kAttnHeads * D + lane] = ep[kAttnHeads * ES + lane];
    }
}

// Where global step `gs` lies: its sequence, its (KV head, pass, timestep) and the step inside that item.
// Items are ordered by sequence, then by gt; prefix[r] = steps of the sequences before r.
struct StepPos { int row, gt, step, nsteps; };
__device__ __forceinline__ StepPos locate_step(const int* prefix, int n_seqs, int gt_count, int64_t gs) {
    int lo = 0, hi = n_seqs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(prefix[mid]) * gt_count <= gs) lo = mid; else hi = mid;
    }
    StepPos r;
    r.row = lo;
    r.nsteps = prefix[lo + 1] - prefix[lo];
    const int rem = static_cast<int>(gs - static_cast<int64_t>(prefix[lo]) * gt_count);
    r.gt = rem / r.nsteps;
    r.step = rem - r.gt * r.nsteps;
    return r;
}

__device__ __forceinline__ int steps_of(int len) { return len > 32 ? (len + 31) >> 5 : 1; }  // an empty row keeps one

// `total` steps in `workers` consecutive ranges whose sizes differ by at most one: the first `rem` ranges hold
// per + 1 steps, the others per.
struct RangeSplit { int64_t per, rem; };
__device__ __forceinline__ RangeSplit make_split(int64_t total, int64_t workers) {
    RangeSplit r;
    if (total < (1LL << 31)) {  // the common case in 32-bit arithmetic
        r.per = static_cast<uint32_t>(total) / static_cast<uint32_t>(workers);
        r.rem = static_cast<uint32_t>(total) - static_cast<uint32_t>(r.per) * static_cast<uint32_t>(workers);
    } else {
        r.per = total / workers;
        r.rem = total - r.per * workers;
    }
    return r;
}
__device__ __forceinline__ int64_t range_start(const RangeSplit& r, int64_t w) { return w * r.per + (w < r.rem ? w : r.rem); }
// the range that holds step x
__device__ __forceinline__ int64_t range_of(const RangeSplit& r, int64_t x) {
    const int64_t head = r.rem * (r.per + 1);  // steps in the longer ranges
    if (x < head) return x / (r.per + 1);
    return r.rem + (x - head) / r.per;         // per >= 1 here, or x < head would hold
}

// DENSE (up to kDenseRows sequences): the work of the whole call is one list of 32-key steps, ordered by item;
// the warps of the grid cut it into equal consecutive ranges, so every warp carries the same number of steps
// whatever the mix of row lengths.  A short item (at most sp.short_steps steps) is never cut: it belongs, whole, to
// the range it starts in.  A warp therefore works on a few pieces: whole items (written straight to the output)
// and at most two cut ones, the item that began before its range (record slot 0) and the one that continues
// after it (slot 1).
// Otherwise: one warp per (unit of unit_keys keys, gt), units enumerated as row * max_units + unit.
template <int W, int NB, bool DENSE>
__global__ void __launch_bounds__(kThreads, (W == 2 ? (NB == 1 ? SPK_STREAM_MINB : 4) : (NB == 1 ? SPK_STREAM_MINB4 : 3)))
attn_stream_kernel(const AttnParams p, const StreamParams sp) {
    using S = StreamSmem<W>;
    constexpr int D = S::D;
    __shared__ __align__(16) uint32_t ring_all[kWarps][S::STAGES][S::TILE_WORDS];
    __shared__ __align__(16) uint32_t x_all[kWarps][W * kXGroup];
    __shared__ int32_t tbl_all[kWarps][kTblMax];
    __shared__ uint32_t rlut[D + 1];  // rlut[i] = {hi, lo} fp16 of 2^14 exp(-(D - i) scale)
    __shared__ int prefix[DENSE ? kDenseRows + 1 : 1];
    __shared__ int lens_s[DENSE ? kDenseRows : 1];
    __shared__ int warp_sums[kWarps];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_seqs = static_cast<int>(p.n_seqs);

    // ---- set-up shared by the CTA: the step prefix and the weight table -----------------------------------
    if (DENSE) {
        // thread t owns rows [t R, (t+1) R): lengths to shared memory, step counts into an exclusive prefix
        const int R = (n_seqs + kThreads - 1) / kThreads;
        const int r0 = threadIdx.x * R;
        int local = 0;
        for (int i = 0; i < R; ++i) {
            const int r = r0 + i;
            if (r < n_seqs) {
                const int raw = __ldg(p.lens + r);
                const int len = clamp_len(raw, p.max_keys);
                if (raw != len && blockIdx.x == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
                lens_s[r] = len;
                local += steps_of(len);
            }
        }
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_sums[warp] = incl;
        for (int i = threadIdx.x; i <= D; i += kThreads) {
            const float wv = ldexpf(expf(-static_cast<float>(D - i) * p.scale), kScaleLog2);
            const __half hi = __float2half_rn(wv);
            const __half lo = __float2half_rn((wv - __half2float(hi)) * 2048.0f);
            rlut[i] = static_cast<uint32_t>(__half_as_ushort(hi)) | (static_cast<uint32_t>(__half_as_ushort(lo)) << 16);
        }
        __syncthreads();
        int run = incl - local;
        for (int w = 0; w < warp; ++w) run += warp_sums[w];
        if (threadIdx.x == 0) prefix[0] = 0;
        for (int i = 0; i < R; ++i) {
            const int r = r0 + i;
            if (r < n_seqs) {
                run += steps_of(lens_s[r]);
                prefix[r + 1] = run;
            }
        }
    } else {
        for (int i = threadIdx.x; i <= D; i += kThreads) {
            const float wv = ldexpf(expf(-static_cast<float>(D - i) * p.scale), kScaleLog2);
            const __half hi = __float2half_rn(wv);
            const __half lo = __float2half_rn((wv - __half2float(hi)) * 2048.0f);
            rlut[i] = static_cast<uint32_t>(__half_as_ushort(hi)) | (static_cast<uint32_t>(__half_as_ushort(lo)) << 16);
        }
    }
    __syncthreads();
    // the combine pass (if one follows) may be scheduled from here on; it waits for this grid's completion itself
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    uint32_t* ring = &ring_all[warp][0][0];
    uint32_t* xb = x_all[warp];
    int32_t* tbl = tbl_all[warp];
    const int64_t worker = static_cast<int64_t>(blockIdx.x) * kWarps + warp;

    if (DENSE) {
        if (worker >= sp.workers) return;
        const int64_t total = static_cast<int64_t>(prefix[n_seqs]) * sp.gt;
        // this warp's range of the step list; a short item belongs, whole, to the range it starts in
        const RangeSplit split = make_split(total, sp.workers);
        int64_t gs = range_start(split, worker);
        const int64_t gend = worker + 1 < sp.workers ? range_start(split, worker + 1) : total;
        bool first = true;
        while (gs < gend) {
            const StepPos at = locate_step(prefix, n_seqs, sp.gt, gs);
            const bool is_short = at.nsteps <= sp.short_steps;
            if (first && is_short && at.step > 0) {  // started in the previous range: not ours
                gs += at.nsteps - at.step;
                first = false;
                continue;
            }
            first = false;
            const int last = is_short ? at.nsteps
                                      : static_cast<int>(min(static_cast<int64_t>(at.nsteps), at.step + (gend - gs)));
            const int len = lens_s[at.row];
            const bool whole = at.step == 0 && last == at.nsteps;
            float* rec = sp.dense_ws + (2 * worker + (at.step > 0 ? 0 : 1)) * sp.rec;
            stream_piece<W, NB>(p, sp, at.row, at.gt, 32 * at.step, min(len, 32 * last), whole, rec, ring, xb, tbl, rlut, lane);
            gs += last - at.step;
        }
    } else {
        const int gt = static_cast<int>(worker % sp.gt);
        const int64_t j = worker / sp.gt;
        if (j >= static_cast<int64_t>(n_seqs) * sp.max_units) return;
        const int row = static_cast<int>(j / sp.max_units);
        const int unit = static_cast<int>(j - static_cast<int64_t>(row) * sp.max_units);
        const int raw = __ldg(p.lens + row);
        const int len = clamp_len(raw, p.max_keys);
        if (raw != len && gt == 0 && unit == 0 && lane == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
        const int n_units = units_of(len, sp.unit_log2);
        if (unit >= n_units) return;
        const int key0 = unit << sp.unit_log2;
        float* rec = p.ws + ((static_cast<int64_t>(row) * sp.gt + gt) * sp.max_units + unit) * sp.rec;
        stream_piece<W, NB>(p, sp, row, gt, key0, min(len, key0 + (1 << sp.unit_log2)), n_units == 1, rec, ring, xb, tbl,
                            rlut, lane);
    }
}

// ---------------------------------------------------------------------------------------------------------
// The same attention on the fifth-generation tensor cores (tcgen05), for head_dim 64 and 16-bit outputs.
//
// What changes against the mma.sync form above is who touches the operands.  There every thread of a warp had to
// receive the K rows of its eight keys and the V words of its fragment through the shared-memory crossbar (about
// 50 wavefronts per 32 keys, the limit of that form).  Here a lane owns ONE key:
//   * it reads the key's K row once and scores it against all query heads of the group (q lives in registers,
//     the same in every lane): popc(q_h & k), exact;
//   * the weight of (head, key) is looked up as a 32-bit fixed-point number round(2^32 exp((s - popc(q)) scale))
//     and written to shared memory as it is: its four bytes are four base-256 digits, i.e. four columns of the
//     right operand [keys x (8 heads x 4 digits)];
//   * the key's 64 V bits are expanded to 64 bytes (bit e of a byte becomes the byte value 2^e, two logic
//     operations per four channels) and written as one row of the left operand [channels x keys].
// One tcgen05.mma.kind::i8 (M = 128: 64 channels, a row of ones for the weight totals, padding; N = 32; K = 32
// keys), issued by one lane, multiplies them straight out of shared memory into an int32 accumulator in tensor
// memory: sums are exact integers, digits are recombined once per unit.  Both operands are stored "MN-major"
// without swizzle: [16-byte group of rows/columns][key][16 bytes], so a lane writes whole 16-byte chunks at
// consecutive addresses.
// Each warp still runs its own unit, with two operand stages so that the next 32 keys are prepared while the
// tensor core works; a warp waits on its stage's mbarrier (tcgen05.commit) before it overwrites the stage.
// Accumulator rows live in TMEM lanes, and a warp can only read the 32 lanes of its own quarter, so the
// epilogue is CTA-wide: after a barrier, warps 0..2 move all four accumulators to shared memory and every warp
// finishes its own unit from there.
// ---------------------------------------------------------------------------------------------------------
constexpr int kTcStages = 2;
constexpr int kTcRing = 4;                 // 64-key tiles of raw K/V rows in flight per warp
constexpr int kTcABytes = 8 * 32 * 16;     // left operand stage: 8 row groups x 32 keys x 16 bytes
constexpr int kTcBBytes = 2 * 32 * 16;     // right operand stage: 2 column groups x 32 keys x 16 bytes
constexpr int kTcRingWords = 2 * kTileKeys * 2;  // K rows then V rows of a 64-key tile, two words per row
constexpr int kTcWaitLimit = 1 << 20;      // polls of an mbarrier before a warp gives up and flags the status word
constexpr int kTcSmemBytes = kWarps * kTcStages * (kTcABytes + kTcBBytes) + kWarps * kTcRing * kTcRingWords * 4 +
                             kWarps * kTblMax * 4 + (kDenseRows + 1) * 4 + kDenseRows * 4 + 128 * 4 + 256;

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) { return static_cast<uint32_t>(__cvta_generic_to_shared(ptr)); }

// Shared-memory matrix descriptor, no swizzle: start address, byte distance between 8-key groups (leading),
// byte distance between 16-byte row/column groups (stride).
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((saddr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    for (int it = 0; it < kTcWaitLimit && !done; ++it)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                   "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                   "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads, 3)
attn_tc_kernel(const AttnParams p, const StreamParams sp) {
    constexpr int D = 64, W = 2;
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t* a_all = tc_smem;                                                   // [warp][stage][kTcABytes]
    uint8_t* b_all = a_all + kWarps * kTcStages * kTcABytes;                    // [warp][stage][kTcBBytes]
    uint32_t* ring_all = reinterpret_cast<uint32_t*>(b_all + kWarps * kTcStages * kTcBBytes);  // [warp][kTcRing][kTcRingWords]
    int32_t* tbl_all = reinterpret_cast<int32_t*>(ring_all + kWarps * kTcRing * kTcRingWords);
    int* prefix = tbl_all + kWarps * kTblMax;                                   // [kDenseRows + 1]
    int* lens_s = prefix + kDenseRows + 1;                                      // [kDenseRows]
    uint32_t* rlut = reinterpret_cast<uint32_t*>(lens_s + kDenseRows);          // [D + 1] (128 reserved)
    uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(rlut + 128) + 7) & ~uintptr_t(7));  // [warp][stage]
    uint32_t* misc = reinterpret_cast<uint32_t*>(bars + kWarps * kTcStages);    // [0] TMEM base, [1..4] warp sums

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_seqs = static_cast<int>(p.n_seqs);

    // ---- set-up shared by the CTA ------------------------------------------------------------------------
    {
        const int R = (n_seqs + kThreads - 1) / kThreads;
        const int r0 = threadIdx.x * R;
        int local = 0;
        for (int i = 0; i < R; ++i) {
            const int r = r0 + i;
            if (r < n_seqs) {
                const int raw = __ldg(p.lens + r);
                const int len = clamp_len(raw, p.max_keys);
                if (raw != len && blockIdx.x == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
                lens_s[r] = len;
                local += units_of(len, sp.unit_log2);
            }
        }
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) misc[1 + warp] = incl;
        // rlut[i]: the weight for bound - score = D - i as a 32-bit fixed-point number (2^32 stands for 1)
        for (int i = threadIdx.x; i <= D; i += kThreads) {
            const float wv = expf(-static_cast<float>(D - i) * p.scale) * 4294967296.0f;
            rlut[i] = wv >= 4294967040.0f ? 0xFFFFFFFFu : static_cast<uint32_t>(__float2uint_rn(wv));
        }
        // constant half of the left operand stages: row group 4 holds the row of ones (byte 0 of its 16), 5..7 zeros
        for (int i = threadIdx.x; i < kWarps * kTcStages * 4 * 32; i += kThreads) {
            const int buf = i / (4 * 32), rest = i - buf * (4 * 32);
            const int grp = 4 + rest / 32, key = rest & 31;
            *reinterpret_cast<uint4*>(a_all + buf * kTcABytes + grp * 512 + key * 16) = make_uint4(grp == 4 ? 1u : 0u, 0u, 0u, 0u);
        }
        if (threadIdx.x < kWarps * kTcStages)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bars + threadIdx.x)));
        if (warp == 0) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(misc)), "r"(32 * kWarps));
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        int run = incl - local;
        for (int w = 0; w < warp; ++w) run += static_cast<int>(misc[1 + w]);
        if (threadIdx.x == 0) prefix[0] = 0;
        for (int i = 0; i < R; ++i) {
            const int r = r0 + i;
            if (r < n_seqs) {
                run += units_of(lens_s[r], sp.unit_log2);
                prefix[r + 1] = run;
            }
        }
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t tmem_base = misc[0];

    // ---- this warp's unit ----------------------------------------------------------------------------------
    const int64_t worker = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
    const int gt = static_cast<int>(worker % sp.gt);
    const int64_t j = worker / sp.gt;
    bool has_unit = j < prefix[n_seqs];
    int row = 0, unit = 0, len = 0;
    if (has_unit) {
        int lo = 0, hi = n_seqs;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= j) lo = mid; else hi = mid;
        }
        row = lo;
        unit = static_cast<int>(j) - prefix[lo];
        len = lens_s[lo];
    }
    const int t = gt % p.T;
    const int gp = gt / p.T;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * kAttnHeads;
    const int nh = min(kAttnHeads, p.n_rep - pass * kAttnHeads);
    const int n_units = units_of(len, sp.unit_log2);
    const int key0 = unit << sp.unit_log2;
    const int kend = min(len, key0 + (1 << sp.unit_log2));
    const int nkeys = has_unit ? max(kend - key0, 0) : 0;
    const int ntiles = (nkeys + kTileKeys - 1) / kTileKeys;
    const int nsteps = (nkeys + 31) >> 5;
    bool failed = false;

    if (nsteps > 0) {
        // block-table entries of the unit's pages, checked once
        int32_t* tbl = tbl_all + warp * kTblMax;
        const int page0 = key0 >> p.bs_log2;
        const int npages = ((kend - 1) >> p.bs_log2) - page0 + 1;
        {
            const int32_t* table = p.tables + row * p.sbt_n + page0;
            for (int i = lane; i < npages; i += 32) {
                int32_t ph = __ldg(table + i);
                if (static_cast<uint32_t>(ph) >= static_cast<uint32_t>(p.num_blocks)) {
                    spk_flag(p.status, SPK_STATUS_BAD_BLOCK);
                    ph = 0;
                }
                tbl[i] = ph;
            }
        }
        // query words of every head of the group (the same in all lanes) and the table position of each head
        uint32_t q0[kAttnHeads], q1[kAttnHeads];
        int hb[kAttnHeads];  // rlut[hb[h] + score] is head h's weight
#pragma unroll
        for (int h = 0; h < kAttnHeads; ++h) {
            q0[h] = q1[h] = 0u;
            if (h < nh) {
                const uint32_t* qp = p.q + t * p.sq_t + row * p.sq_n + (h0 + h) * p.sq_h;
                q0[h] = __ldg(qp);
                q1[h] = __ldg(qp + 1);
            }
            hb[h] = D - __popc(q0[h]) - __popc(q1[h]);
        }
        __syncwarp();

        // raw K/V rows: 64-key tiles through a cp.async ring (lane l copies keys 2l, 2l+1: 16 bytes of K, 16 of V)
        uint32_t* ring = ring_all + warp * kTcRing * kTcRingWords;
        const uint32_t ring_addr = smem_u32(ring) + lane * 16;
        const uint32_t* kbase = p.k + t * p.sk_t + g * p.sk_h;
        const uint32_t* vbase = p.v + t * p.sv_t + g * p.sv_h;
        const int bs_mask = (1 << p.bs_log2) - 1;
        const int last_page = npages - 1;
        int issue_key = key0 + 2 * lane;
        uint32_t issue_stage = 0;
        auto issue = [&]() {
            const int bytes = issue_key < kend ? 16 : 0;
            const int pl = min((issue_key >> p.bs_log2) - page0, last_page);
            const int off = tbl[pl] * p.sk_blk + (issue_key & bs_mask) * W;
            cp_async16(ring_addr + issue_stage, kbase + off, bytes);
            cp_async16(ring_addr + issue_stage + kTileKeys * W * 4, vbase + off, bytes);
            issue_key += kTileKeys;
            issue_stage = issue_stage == (kTcRing - 1) * kTcRingWords * 4 ? 0u : issue_stage + kTcRingWords * 4;
        };
#pragma unroll
        for (int s = 0; s < kTcRing - 1; ++s) {
            if (s < ntiles) issue();
            cp_async_commit();
        }

        uint8_t* a_st = a_all + warp * kTcStages * kTcABytes;
        uint8_t* b_st = b_all + warp * kTcStages * kTcBBytes;
        const uint32_t bar0 = smem_u32(bars + warp * kTcStages);
        // s32 accumulator, u8 x u8, both operands MN-major, N = 32, M = 128
        constexpr uint32_t idesc = (2u << 4) | (1u << 15) | (1u << 16) | ((32u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t d_tmem = tmem_base + 32 * warp;

        const uint32_t* tile_words = ring;
        for (int step = 0; step < nsteps; ++step) {
            const int half = step & 1;
            if (half == 0) {
                cp_async_wait<kTcRing - 2>();
                __syncwarp();
                if ((step >> 1) + kTcRing - 1 < ntiles) issue();
                cp_async_commit();
            }
            // this lane's key: its K row scored against every head, its V row expanded
            const uint2 kr = *reinterpret_cast<const uint2*>(tile_words + (32 * half + lane) * W);
            const uint2 vr = *reinterpret_cast<const uint2*>(tile_words + kTileKeys * W + (32 * half + lane) * W);
            const bool live = 32 * step + lane < nkeys;
            uint32_t wq[kAttnHeads];
#pragma unroll
            for (int h = 0; h < kAttnHeads; ++h) {
                const int s = __popc(q0[h] & kr.x) + __popc(q1[h] & kr.y);
                wq[h] = (h < nh && live) ? rlut[hb[h] + s] : 0u;
            }
            const int stage = step & (kTcStages - 1);
            if (step >= kTcStages && !failed) {
                // the MMA that read this stage two steps ago must have finished
                if (!mbar_wait(bar0 + stage * 8, ((step / kTcStages) - 1) & 1)) failed = true;
            }
            uint8_t* a_dst = a_st + stage * kTcABytes + lane * 16;
            uint8_t* b_dst = b_st + stage * kTcBBytes + lane * 16;
            *reinterpret_cast<uint4*>(b_dst) = make_uint4(wq[0], wq[1], wq[2], wq[3]);
            *reinterpret_cast<uint4*>(b_dst + 512) = make_uint4(wq[4], wq[5], wq[6], wq[7]);
#pragma unroll
            for (int grp = 0; grp < 4; ++grp) {
                // bytes 2 grp and 2 grp + 1 of the 8-byte V row: 16 channels -> 16 bytes, bit e of a byte -> value 2^e
                const uint32_t word = grp < 2 ? vr.x : vr.y;
                const uint32_t r0 = prmt(word, 0u, (grp & 1) ? 0x2222u : 0x0000u);
                const uint32_t r1 = prmt(word, 0u, (grp & 1) ? 0x3333u : 0x1111u);
                *reinterpret_cast<uint4*>(a_dst + grp * 512) =
                    make_uint4(r0 & 0x08040201u, r0 & 0x80402010u, r1 & 0x08040201u, r1 & 0x80402010u);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && !failed) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = tc_desc(smem_u32(a_st + stage * kTcABytes), 128, 512);
                const uint64_t db = tc_desc(smem_u32(b_st + stage * kTcBBytes), 128, 512);
                const uint32_t accumulate = step > 0 ? 1u : 0u;
                const uint32_t zero = 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
                    ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                             ::"r"(bar0 + stage * 8) : "memory");
            }
            if (half == 1) tile_words = ((step >> 1) % kTcRing == kTcRing - 1) ? ring : tile_words + kTcRingWords;
        }
        cp_async_wait<0>();
        // the last commit covers every MMA this warp issued
        const int last = nsteps - 1;
        if (!failed && !mbar_wait(bar0 + (last & (kTcStages - 1)) * 8, (last / kTcStages) & 1)) failed = true;
        if (failed && lane == 0) spk_flag(p.status, SPK_STATUS_DEVICE_WAIT_EXPIRED);
    }

    // ---- CTA-wide epilogue: accumulators TMEM -> shared memory, then every warp finishes its own unit ---------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // raw[acc][row 0..63][32 columns] int32, 16-byte chunks XOR-swizzled by row, over the (now idle) left operand
    // stages; totals[acc][32] over the right operand stages
    int32_t* raw = reinterpret_cast<int32_t*>(a_all);
    int32_t* totals = reinterpret_cast<int32_t*>(b_all);
    if (warp < 3) {
#pragma unroll 1
        for (int acc = 0; acc < kWarps; ++acc) {
            uint32_t r[32];
            tmem_ld32(tmem_base + (static_cast<uint32_t>(32 * warp) << 16) + 32 * acc, r);
            if (warp < 2) {
                const int rr = 32 * warp + lane;
                int32_t* dst = raw + (acc * 64 + rr) * 32;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(dst + 4 * (c ^ (rr & 7))) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
            } else if (lane == 0) {
#pragma unroll
                for (int c = 0; c < 32; ++c) totals[acc * 32 + c] = static_cast<int32_t>(r[c]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32 * kWarps));
    if (!has_unit || unit >= n_units) return;

    // lane -> (head, quarter of the channels); digits d0..d3 of a sum recombine as d0 + 2^8 d1 + 2^16 d2 + 2^24 d3
    const int hh = lane >> 2, qc = lane & 3;
    auto digits = [](const int4 d) {
        return static_cast<float>(d.x) + 256.0f * static_cast<float>(d.y) + 65536.0f * static_cast<float>(d.z) +
               16777216.0f * static_cast<float>(d.w);
    };
    float vals[16];
    float tot = 0.0f;
    if (nsteps > 0 && !failed) {
        tot = digits(*reinterpret_cast<const int4*>(totals + warp * 32 + 4 * hh));
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const int ch = 16 * qc + c;
            const int4 d = *reinterpret_cast<const int4*>(raw + (warp * 64 + ch) * 32 + 4 * (hh ^ (ch & 7)));
            // channel ch was stored as 2^(ch % 8)
            vals[c] = digits(d) * __uint_as_float(static_cast<uint32_t>(127 - (ch & 7)) << 23);
        }
    } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) vals[c] = 0.0f;
    }
    if (n_units == 1) {
        if (hh < nh) {
            const float inv = tot > 0.0f ? 1.0f / tot : 0.0f;
            const int64_t idx = t * p.so_t + row * p.so_n + (h0 + hh) * p.so_h + 16 * qc;
            if (p.out_dtype == SPK_BF16) {
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + idx;
                if (sp.out_vec) {
#pragma unroll
                    for (int c = 0; c < 16; c += 8) {
                        union { uint4 u; __nv_bfloat16 e[8]; } pk;
#pragma unroll
                        for (int i = 0; i < 8; ++i) pk.e[i] = __float2bfloat16_rn(vals[c + i] * inv);
                        *reinterpret_cast<uint4*>(dst + c) = pk.u;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 16; ++c) dst[c] = __float2bfloat16_rn(vals[c] * inv);
                }
            } else {
                __half* dst = static_cast<__half*>(p.out) + idx;
                if (sp.out_vec) {
#pragma unroll
                    for (int c = 0; c < 16; c += 8) {
                        union { uint4 u; __half e[8]; } pk;
#pragma unroll
                        for (int i = 0; i < 8; ++i) pk.e[i] = __float2half_rn(vals[c + i] * inv);
                        *reinterpret_cast<uint4*>(dst + c) = pk.u;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 16; ++c) dst[c] = __float2half_rn(vals[c] * inv);
                }
            }
        }
    } else {
        // partial record; sums and totals both carry the factor 2^32, scaled down here to keep fp32 sums of many
        // records well inside the format
        constexpr float kDown = 1.0f / 4294967296.0f;
        float* rec = p.ws + ((static_cast<int64_t>(row) * sp.gt + gt) * sp.max_units + unit) * sp.rec;
#pragma unroll
        for (int c = 0; c < 16; c += 4)
            *reinterpret_cast<float4*>(rec + hh * D + 16 * qc + c) =
                make_float4(vals[c] * kDown, vals[c + 1] * kDown, vals[c + 2] * kDown, vals[c + 3] * kDown);
        if (qc == 0) rec[kAttnHeads * D + hh] = tot * kDown;
    }
}

// Sums the partial records of one (sequence, KV head, pass, timestep) in key order and divides.  Items that one
// warp finished alone were written by the main kernel and are skipped.  A thread owns four channels of one head;
// the records' values are fetched eight records at a time (independent loads) and added in record order.
// MAXW: the most records a thread fetches together.  Sixteen shortens the pass for items of many pieces but costs
// registers (128 against 80), which the many small CTAs of a large batch pay for in residency; the host picks
// sixteen for calls of up to 512 items.
template <int MAXW>
__global__ void __launch_bounds__(128)
attn_stream_combine_kernel(const AttnParams p, const StreamParams sp, int D) {
    // a following launch that asked to overlap (it waits for this grid before it touches q, K/V or the records)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t item = blockIdx.x;  // row * gt_count + gt
    const int gt = static_cast<int>(item % sp.gt);
    const int64_t row = item / sp.gt;
    const int len = clamp_len(__ldg(p.lens + row), p.max_keys);
    if (sp.dense) {
        if (steps_of(len) <= sp.short_steps) return;  // never cut
    } else if (units_of(len, sp.unit_log2) <= 1) {
        return;
    }
    const int t = gt % p.T;
    const int gp = gt / p.T;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * kAttnHeads;
    const int nh = min(kAttnHeads, p.n_rep - pass * kAttnHeads);
    // records of this item: count, and where record i lies.  All of it follows from the lengths, so it is worked
    // out here, while the main kernel still runs.
    int n_rec;
    int64_t first = 0;
    if (sp.dense) {
        // steps of the rows before this one, and of all rows (the main kernel's step prefix, recomputed)
        __shared__ int red[2][4];
        int before = 0, all = 0;
        for (int r = threadIdx.x; r < static_cast<int>(p.n_seqs); r += blockDim.x) {
            const int st = steps_of(clamp_len(__ldg(p.lens + r), p.max_keys));
            all += st;
            if (r < row) before += st;
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            before += __shfl_xor_sync(0xffffffffu, before, o);
            all += __shfl_xor_sync(0xffffffffu, all, o);
        }
        if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = before; red[1][threadIdx.x >> 5] = all; }
        __syncthreads();
        before = red[0][0] + red[0][1] + red[0][2] + red[0][3];
        all = red[1][0] + red[1][1] + red[1][2] + red[1][3];
        // the item's interval of the step list; piece i belongs to worker first + i: the first one started the
        // item (slot 1), the others continued it (slot 0)
        const int64_t total = static_cast<int64_t>(all) * sp.gt;
        const RangeSplit split = make_split(total, sp.workers);
        const int nsteps = steps_of(len);
        const int64_t g0 = static_cast<int64_t>(before) * sp.gt + static_cast<int64_t>(gt) * nsteps;
        first = range_of(split, g0);
        n_rec = static_cast<int>(range_of(split, g0 + nsteps - 1) - first) + 1;
        if (n_rec <= 1) return;
    } else {
        n_rec = units_of(len, sp.unit_log2);
    }
    // the records are complete once the main kernel's grid has finished and flushed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    auto record = [&](int u) -> const float* {
        return sp.dense ? sp.dense_ws + (2 * (first + u) + (u == 0 ? 1 : 0)) * sp.rec : p.ws + (item * sp.max_units + u) * sp.rec;
    };
    const int quads = D / 4;
    // (head, four channels) pairs of the item over the threads of its gridDim.y CTAs: one pair per thread
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < nh * quads; idx += gridDim.y * blockDim.x) {
        const int hh = idx / quads;
        const int d = 4 * (idx - hh * quads);
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float l = 0.0f;
        // records fetched together (independent loads), added in record order; as many in flight as the item has
        // pieces, up to MAXW (indices past the last piece re-read the last record and are not added)
        auto add_records = [&](auto width) {
            constexpr int kInFlight = decltype(width)::value;
            for (int u0 = 0; u0 < n_rec; u0 += kInFlight) {
                float4 v[kInFlight];
                float w[kInFlight];
#pragma unroll
                for (int i = 0; i < kInFlight; ++i) {
                    const float* rec = record(min(u0 + i, n_rec - 1));
                    v[i] = *reinterpret_cast<const float4*>(rec + hh * D + d);
                    w[i] = rec[kAttnHeads * D + hh];
                }
#pragma unroll
                for (int i = 0; i < kInFlight; ++i)
                    if (u0 + i < n_rec) { a.x += v[i].x; a.y += v[i].y; a.z += v[i].z; a.w += v[i].w; l += w[i]; }
            }
        };
        if (n_rec <= 4) add_records(std::integral_constant<int, 4>{});
        else if (MAXW <= 8 || n_rec <= 8) add_records(std::integral_constant<int, 8>{});
        else add_records(std::integral_constant<int, MAXW>{});
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        const int64_t o = t * p.so_t + row * p.so_n + (h0 + hh) * p.so_h + d;
        const float r4[4] = {a.x * inv, a.y * inv, a.z * inv, a.w * inv};
        if (sp.out_vec) {  // rows 16-byte aligned: the four channels leave as one store
            if (p.out_dtype == SPK_F32) {
                *reinterpret_cast<float4*>(static_cast<float*>(p.out) + o) = make_float4(r4[0], r4[1], r4[2], r4[3]);
            } else if (p.out_dtype == SPK_BF16) {
                union { uint2 u; __nv_bfloat162 h[2]; } pk;
                pk.h[0] = __floats2bfloat162_rn(r4[0], r4[1]);
                pk.h[1] = __floats2bfloat162_rn(r4[2], r4[3]);
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + o) = pk.u;
            } else {
                union { uint2 u; __half2 h[2]; } pk;
                pk.h[0] = __floats2half2_rn(r4[0], r4[1]);
                pk.h[1] = __floats2half2_rn(r4[2], r4[3]);
                *reinterpret_cast<uint2*>(static_cast<__half*>(p.out) + o) = pk.u;
            }
            continue;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (p.out_dtype == SPK_F32) static_cast<float*>(p.out)[o + i] = r4[i];
            else if (p.out_dtype == SPK_BF16) static_cast<__nv_bfloat16*>(p.out)[o + i] = __float2bfloat16_rn(r4[i]);
            else static_cast<__half*>(p.out)[o + i] = __float2half_rn(r4[i]);
        }
    }
}

static inline int log2_exact(int x) {
    if (x < 1 || (x & (x - 1)) != 0) return -1;
    int l = 0;
    while ((1 << l) < x) ++l;
    return l;
}

template <int W, int NB>
int launch_stream(const AttnParams& p, const StreamParams& sp, int64_t ctas, bool overlap, cudaStream_t stream) {
    // overlap: the caller vouches that lengths and block tables were complete before the PREVIOUS launch on
    // this stream began, so this grid may be placed while that launch still runs (programmatic stream
    // serialisation); the kernel reads nothing else before its griddepcontrol.wait.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    const cudaError_t e = sp.dense ? cudaLaunchKernelEx(&cfg, attn_stream_kernel<W, NB, true>, p, sp)
                                   : cudaLaunchKernelEx(&cfg, attn_stream_kernel<W, NB, false>, p, sp);
    if (e != cudaSuccess) return spk_set_cuda_error(e);
    spk_count_launch();
    return SPK_OK;
}

}  // namespace

static std::atomic<int> g_attn_form{SPK_ATTN_FORM_AUTO};

extern "C" int spk_attn_select_form(int form) {
    if (form < SPK_ATTN_FORM_AUTO || form > SPK_ATTN_FORM_TCGEN05) return SPK_ERR_UNSUPPORTED;
    g_attn_form.store(form, std::memory_order_relaxed);
    return SPK_OK;
}

int spk_attn_selected_form() { return g_attn_form.load(std::memory_order_relaxed); }

// CTAs per SM the main kernel is built for (its __launch_bounds__), by rows of words and weight blocks.
static int stream_ctas_per_sm(int head_dim, bool wide) {
    if (head_dim == 64) return wide ? 4 : SPK_STREAM_MINB;
    return wide ? 3 : SPK_STREAM_MINB4;
}

StreamPlan spk_attn_stream_plan(int T, int64_t n_seqs, int Hq, int Hkv, int head_dim, int block_size,
                                int64_t max_blocks) {
    StreamPlan pl = {};
    const int bs_log2 = log2_exact(block_size);
    if ((head_dim != 64 && head_dim != 128) || bs_log2 < 2 || T < 1 || n_seqs < 1 || Hq < 1 || Hkv < 1 ||
        Hq % Hkv != 0 || max_blocks < 1)
        return pl;
    const int n_rep = Hq / Hkv;
    pl.passes = (n_rep + kAttnHeads - 1) / kAttnHeads;
    const int64_t max_keys = max_blocks * block_size;
    const int64_t gt = static_cast<int64_t>(T) * Hkv * pl.passes;
    pl.rec_floats = static_cast<int64_t>(kAttnHeads) * head_dim + 8;
    const int64_t rec_bytes = pl.rec_floats * static_cast<int64_t>(sizeof(float));

    // unit form (more than kDenseRows sequences, and the tcgen05 form): units of 512..2048 keys; a unit's
    // block-table entries must fit their staging (kTblMax) and a row at most 256 units
    int unit = 512;
    for (int cand = 2048; cand > 512; cand >>= 1) {
        if (cand / block_size > kTblMax) continue;
        const int64_t est = n_seqs * gt * (max_keys / (2 * cand) + 1);
        if (est >= 2 * static_cast<int64_t>(kResidentWarpsTarget)) { unit = cand; break; }
    }
    while ((max_keys + unit - 1) / unit > 256 && unit < 2048 && (2 * unit) / block_size <= kTblMax) unit *= 2;
    if (unit / block_size > kTblMax) return pl;
    const int64_t max_units = (max_keys + unit - 1) / unit;
    if (max_units > 256) return pl;
    if (n_seqs * max_units * gt > (1LL << 33)) return pl;
    pl.unit_keys = unit;
    pl.max_units = static_cast<int>(max_units);
    const int64_t unit_bytes = max_units > 1 ? n_seqs * gt * max_units * rec_bytes : 0;

    // range form (up to kDenseRows sequences): the step list is shared by `workers` warps, at least eight steps
    // each if every row were full, at most what the GPU holds at once; two record slots per worker and the step
    // prefix, needed only if some item can be cut (pl.short_steps)
    pl.dense = n_seqs <= kDenseRows;
    int64_t range_bytes = 0;
    if (pl.dense) {
        const int64_t max_steps = (max_keys + 31) / 32;
        const int64_t all_steps = n_seqs * gt * max_steps;
        const int64_t cap = 148LL * kWarps * stream_ctas_per_sm(head_dim, /*wide=*/false);  // the most any output type uses
        int64_t workers = (all_steps + 7) / 8;
        workers = workers < 1 ? 1 : (workers > cap ? cap : workers);
        pl.workers = workers;
        pl.short_steps = max_steps <= kUncutSteps ? static_cast<int>(max_steps) : kShortSteps;
        pl.cut = max_steps > pl.short_steps;
        if (!pl.cut) {
            // whole items only: a warp per item while the GPU holds them all at once
            const int64_t items = n_seqs * gt;
            if (workers < items) workers = items < cap ? items : cap;
            pl.workers = workers;
        }
        if (pl.cut) range_bytes = workers * 2 * rec_bytes;
    }
    // the tcgen05 form (selectable at head_dim 64) uses the unit records
    const bool unit_form_possible = !pl.dense || head_dim == 64;
    pl.ws_bytes = range_bytes;
    if (unit_form_possible && unit_bytes > pl.ws_bytes) pl.ws_bytes = unit_bytes;
    pl.ok = true;
    return pl;
}

bool spk_attn_stream_layout_ok(const AttnParams& p, int head_dim) {
    const int W = head_dim / 32;
    auto aligned = [](const void* ptr, int64_t a, int64_t b, int64_t c) {
        return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && a % 4 == 0 && b % 4 == 0 && c % 4 == 0;
    };
    // page offsets are formed in 32 bits inside a (timestep, head) slab
    if (static_cast<int64_t>(p.num_blocks) * p.sk_blk > 0x7fffffffLL) return false;
    return p.sk_slot == W && p.sv_slot == W && p.sk_blk >= 0 && p.sv_blk >= 0 &&
           p.sk_blk == p.sv_blk && aligned(p.k, p.sk_t, p.sk_h, p.sk_blk) && aligned(p.v, p.sv_t, p.sv_h, p.sv_blk);
}

static int launch_combine(const AttnParams& p, const StreamParams& sp, int head_dim, cudaStream_t stream) {
    // Launched with programmatic stream serialisation: its CTAs may be placed while the main kernel still
    // runs (the launch latency overlaps), and each waits for the main grid before it reads a record.
    if (p.n_seqs * sp.gt > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p.n_seqs * sp.gt), static_cast<unsigned>((kAttnHeads * (head_dim / 4) + 127) / 128));
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = p.n_seqs * sp.gt <= 512 ? cudaLaunchKernelEx(&cfg, attn_stream_combine_kernel<16>, p, sp, head_dim)
                                                   : cudaLaunchKernelEx(&cfg, attn_stream_combine_kernel<8>, p, sp, head_dim);
    if (e != cudaSuccess) return spk_set_cuda_error(e);
    spk_count_launch();
    return SPK_OK;
}

int spk_attn_stream_launch(const AttnParams& p, const StreamPlan& plan, int head_dim, cudaStream_t stream) {
    StreamParams sp = {};
    sp.unit_log2 = log2_exact(plan.unit_keys);
    sp.max_units = plan.max_units;
    sp.gt = p.T * p.Hkv * plan.passes;
    sp.dense = plan.dense;
    sp.rec = plan.rec_floats;
    sp.short_steps = plan.short_steps;
    const int esize = p.out_dtype == SPK_F32 ? 4 : 2;
    const int per = 16 / esize;
    sp.out_vec = reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && p.so_t % per == 0 && p.so_n % per == 0 && p.so_h % per == 0;
    const bool wide = p.out_dtype == SPK_F32;  // fp32 output: {hi, lo} weights

    // tcgen05 form, on request: head_dim 64, 16-bit output, up to kDenseRows sequences, weights down to e^-16 of the
    // bound.  It is slower than the mma.sync form (the expanded operands cross shared memory twice), so it is never
    // chosen automatically.
    if (spk_attn_selected_form() == SPK_ATTN_FORM_TCGEN05 && head_dim == 64 && !wide && plan.dense &&
        p.scale * 64.0f <= 16.0f) {
        // the kernel's dynamic shared memory is above the default limit: raised once per device
        static std::atomic<bool> raised[64];
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return spk_set_cuda_error(e);
        if (dev < 0 || dev >= 64) return SPK_ERR_UNSUPPORTED;
        if (!raised[dev].load(std::memory_order_acquire)) {
            e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes);
            if (e != cudaSuccess) return spk_set_cuda_error(e);
            raised[dev].store(true, std::memory_order_release);
        }
        const int64_t ctas = (p.n_seqs * plan.max_units * sp.gt + kWarps - 1) / kWarps;
        if (ctas > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
        sp.dense = 0;  // unit records, for the combine pass
        attn_tc_kernel<<<static_cast<unsigned>(ctas), kThreads, kTcSmemBytes, stream>>>(p, sp);
        SPK_CHECK_LAUNCH();
        return plan.max_units > 1 ? launch_combine(p, sp, head_dim, stream) : SPK_OK;
    }

    const bool overlap = p.overlap != 0;
    int64_t ctas;
    bool combine;
    if (plan.dense) {
        // as many warps as this output type keeps resident, within what the plan's workspace allows
        const int64_t resident = 148LL * kWarps * stream_ctas_per_sm(head_dim, wide);
        sp.workers = plan.workers < resident ? plan.workers : resident;
        sp.dense_ws = p.ws;
        ctas = (sp.workers + kWarps - 1) / kWarps;
        combine = plan.cut;
        if (!plan.cut && sp.workers >= p.n_seqs * sp.gt) {
            // Nothing can be cut and the GPU holds a warp per item at once: warp w runs item w whole, whatever the
            // rows' lengths (equal step ranges would hand some warps two ragged items and others none).  That is
            // the unit form with one unit per row, which also needs no step prefix.
            sp.dense = 0;
            sp.unit_log2 = 30;
            sp.max_units = 1;
            ctas = (p.n_seqs * sp.gt + kWarps - 1) / kWarps;
        }
    } else {
        // worst case of the enumeration: every row of max_units units (the surplus warps leave at once)
        ctas = (p.n_seqs * plan.max_units * sp.gt + kWarps - 1) / kWarps;
        combine = plan.max_units > 1;
    }
    if (ctas > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    int rc;
    if (head_dim == 64) rc = wide ? launch_stream<2, 2>(p, sp, ctas, overlap, stream) : launch_stream<2, 1>(p, sp, ctas, overlap, stream);
    else rc = wide ? launch_stream<4, 2>(p, sp, ctas, overlap, stream) : launch_stream<4, 1>(p, sp, ctas, overlap, stream);
    if (rc != SPK_OK) return rc;
    return combine ? launch_combine(p, sp, head_dim, stream) : SPK_OK;
}
