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

namespace {

constexpr int kWarps = 4;          // independent workers per CTA
constexpr int kThreads = 32 * kWarps;
constexpr int kTileKeys = 64;      // keys per pipeline stage: two 32-key MMA tiles
constexpr int kTblMax = 128;       // block-table entries staged per unit (2048 keys of 16-key pages)
constexpr int kDenseRows = 1024;   // up to this many sequences the units are enumerated densely
constexpr int kScaleLog2 = 14;     // weights are kept times 2^14: the largest is 2^14, the smallest used 2^14 e^-24
constexpr float kLoUnscale = 1.0f / 2048.0f;  // the lo half of a weight is stored times 2^11
constexpr int kResidentWarpsTarget = 148 * 20;

struct StreamParams {
    int unit_log2;   // log2 of the keys per unit
    int max_units;   // units of the longest possible row
    int gt;          // T * Hkv * passes: workers per unit
    int dense;       // units enumerated through the prefix sum (n_seqs <= kDenseRows)
    int out_vec;     // output rows may be written with 16-byte stores
    int64_t rec;     // floats per partial record
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

// 32 keys.  kst: their K rows [key][W]; xb: their V rows interleaved by key pair, [pair][2W] half-word
// pairs (word h of a pair = channels 16h..16h+15 of key 2p in the low half, of key 2p+1 in the high half).
// rlut: the weight table positioned so that rlut[score] is this head's weight.
// ALL: every key is live; otherwise keys at or beyond `nlive` get weight zero.
template <int W, int NB, bool ALL>
__device__ __forceinline__ void tile_compute(const uint32_t* kst, const uint32_t* xb, const uint32_t (&qw)[W],
                                             const uint32_t* rlut, int nlive, uint32_t m_lo, uint32_t m_hi,
                                             uint32_t c_hi, const uint32_t (&ones)[4], int tig,
                                             float (&acc)[NB][2 * W + 1][4]) {
    constexpr int MB = 2 * W;  // blocks of 16 channels
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
        uint32_t xa[MB], xc[MB];
        load_words<MB>(xb + (8 * ks + tig) * MB, xa);
        load_words<MB>(xb + (8 * ks + 4 + tig) * MB, xc);
#pragma unroll
        for (int j = 0; j < MB; ++j) {
            const uint32_t a[4] = {xa[j] & m_lo, (xa[j] & m_hi) | c_hi, xc[j] & m_lo, (xc[j] & m_hi) | c_hi};
            mma16816(acc[0][j], a, bh[0], bh[1]);
            if (NB == 2) mma16816(acc[NB - 1][j], a, bl[0], bl[1]);
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
#define SPK_STREAM_MINB 5
#endif

template <int W, int NB, bool DENSE>
__global__ void __launch_bounds__(kThreads, (W == 2 ? (NB == 1 ? SPK_STREAM_MINB : 4) : (NB == 1 ? 4 : 3)))
attn_stream_kernel(const AttnParams p, const StreamParams sp) {
    constexpr int D = 32 * W;
    constexpr int MB = 2 * W;
    constexpr int STAGES = W == 2 ? 4 : 3;             // 64-key tiles in flight per warp
    constexpr int HALF_WORDS = kTileKeys * W;          // words of a tile's K rows (and of its V rows)
    constexpr int TILE_WORDS = 2 * HALF_WORDS;         // K rows then V rows
    constexpr int TILE_BYTES = TILE_WORDS * 4;
    constexpr int ES = D + 4;                          // row stride of the epilogue's transposition buffer
    static_assert(STAGES * TILE_WORDS >= kAttnHeads * ES + 8, "the epilogue reuses the warp's ring");
    __shared__ __align__(16) uint32_t ring_all[kWarps][STAGES][TILE_WORDS];
    __shared__ __align__(16) uint32_t x_all[kWarps][HALF_WORDS];
    __shared__ int32_t tbl_all[kWarps][kTblMax];
    __shared__ uint32_t rlut[D + 1];  // rlut[i] = {hi, lo} fp16 of 2^14 exp(-(D - i) scale)
    __shared__ int prefix[DENSE ? kDenseRows + 1 : 1];
    __shared__ int lens_s[DENSE ? kDenseRows : 1];
    __shared__ int warp_sums[kWarps];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int gid = lane >> 2;  // MMA column = query head; MMA rows gid and gid + 8 = channels
    const int tig = lane & 3;
    const int n_seqs = static_cast<int>(p.n_seqs);

    // ---- set-up shared by the CTA: unit enumeration and the weight table --------------------------------
    if (DENSE) {
        // thread t owns rows [t R, (t+1) R): lengths to shared memory, unit counts into an exclusive prefix
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
                run += units_of(lens_s[r], sp.unit_log2);
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

    // ---- this warp's work: (row, unit) from the worker index, (KV head, pass, timestep) from its remainder ----
    const int64_t worker = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
    const int gt = static_cast<int>(worker % sp.gt);
    const int64_t j = worker / sp.gt;
    int row, unit, len;
    if (DENSE) {
        if (j >= prefix[n_seqs]) return;
        int lo = 0, hi = n_seqs;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= j) lo = mid; else hi = mid;
        }
        row = lo;
        unit = static_cast<int>(j) - prefix[lo];
        len = lens_s[lo];
    } else {
        if (j >= static_cast<int64_t>(n_seqs) * sp.max_units) return;
        row = static_cast<int>(j / sp.max_units);
        unit = static_cast<int>(j - static_cast<int64_t>(row) * sp.max_units);
        const int raw = __ldg(p.lens + row);
        len = clamp_len(raw, p.max_keys);
        if (raw != len && gt == 0 && unit == 0 && lane == 0) spk_flag(p.status, SPK_STATUS_BAD_SEQ_LEN);
    }
    const int t = gt % p.T;
    const int gp = gt / p.T;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * kAttnHeads;
    const int nh = min(kAttnHeads, p.n_rep - pass * kAttnHeads);

    const int n_units = units_of(len, sp.unit_log2);
    if (unit >= n_units) return;
    const int key0 = unit << sp.unit_log2;
    const int kend = min(len, key0 + (1 << sp.unit_log2));
    const int nkeys = max(kend - key0, 0);
    const int ntiles = (nkeys + kTileKeys - 1) / kTileKeys;

    // block-table entries of the unit's pages, checked once
    int32_t* tbl = tbl_all[warp];
    const int page0 = key0 >> p.bs_log2;
    const int npages = nkeys > 0 ? ((kend - 1) >> p.bs_log2) - page0 + 1 : 0;
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
    // query words of this thread's head and their popcount (the softmax bound)
    uint32_t qw[W];
    int cmax = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) {
        qw[w] = gid < nh ? __ldg(p.q + t * p.sq_t + row * p.sq_n + (h0 + gid) * p.sq_h + w) : 0u;
        cmax += __popc(qw[w]);
    }
    const uint32_t* my_rlut = rlut + (D - cmax);
    __syncwarp();

    // ---- copies: a lane moves 16 bytes of K and the same 16 bytes of V per 32 (W = 2: 64) keys ------------
    // W = 2: lane l copies keys 2l, 2l+1 of the 64-key tile (one K and one V segment).
    // W = 4: lane l copies keys l and l + 32 (two K and two V segments).
    uint32_t* ring = &ring_all[warp][0][0];
    const uint32_t ring_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ring)) + lane * 16;
    const uint32_t* kbase = p.k + t * p.sk_t + g * p.sk_h;
    const uint32_t* vbase = p.v + t * p.sv_t + g * p.sv_h;
    const int bs_mask = (1 << p.bs_log2) - 1;
    const int last_page = npages - 1;
    int issue_key = key0 + (W == 2 ? 2 * lane : lane);  // this lane's first key of the next tile to copy
    uint32_t issue_stage = 0;                           // byte offset of that tile's stage in the ring
    auto issue = [&]() {
#pragma unroll
        for (int c = 0; c < (W == 2 ? 1 : 2); ++c) {
            const int key = issue_key + 32 * c;
            const int bytes = key < kend ? 16 : 0;
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

    // masks of this thread's two channel rows (bits gid and gid + 8 of every half-word)
    const uint32_t m_lo = 0x00010001u << gid;
    const uint32_t m_hi = 0x01000100u << gid;
    const uint32_t c_hi = gid == 7 ? 0x40004000u : 0u;  // bit 15 travels with a forced bit 14: +2 or -2
    uint32_t ones[4];  // fp16 {1, 1}: the left operand of the weight totals (kept in registers, opaque to the compiler)
#pragma unroll
    for (int i = 0; i < 4; ++i) asm volatile("mov.b32 %0, 0x3C003C00;" : "=r"(ones[i]));

    float acc[NB][MB + 1][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int jb = 0; jb <= MB; ++jb) acc[b][jb][0] = acc[b][jb][1] = acc[b][jb][2] = acc[b][jb][3] = 0.0f;

    uint32_t* xb = x_all[warp];
    const uint32_t* kst = ring;
    int nlive = nkeys;
    for (int tile = 0; tile < ntiles; ++tile) {
        cp_async_wait<STAGES - 2>();  // this tile has landed (the newer STAGES - 2 groups may be in flight)
        __syncwarp();                 // ... for every lane; and every lane is done with the previous tile
        if (tile + STAGES - 1 < ntiles) issue();  // into the stage the previous tile occupied
        cp_async_commit();
        // interleave the V rows of every key pair by half-word: lane = pair
        {
            const uint32_t* vst = kst + HALF_WORDS + lane * 2 * W;
            uint32_t r[2 * W], x[2 * W];
            load_words<2 * W>(vst, r);  // key 2l: words 0..W-1; key 2l+1: words W..2W-1
#pragma unroll
            for (int w = 0; w < W; ++w) {
                x[2 * w] = prmt(r[w], r[W + w], 0x5410);
                x[2 * w + 1] = prmt(r[w], r[W + w], 0x7632);
            }
#pragma unroll
            for (int i = 0; i < 2 * W; i += 4)
                *reinterpret_cast<uint4*>(xb + lane * 2 * W + i) = make_uint4(x[i], x[i + 1], x[i + 2], x[i + 3]);
        }
        __syncwarp();
        if (nlive >= kTileKeys) {
            tile_compute<W, NB, true>(kst, xb, qw, my_rlut, 32, m_lo, m_hi, c_hi, ones, tig, acc);
            tile_compute<W, NB, true>(kst + 32 * W, xb + 32 * W, qw, my_rlut, 32, m_lo, m_hi, c_hi, ones, tig, acc);
        } else {
            tile_compute<W, NB, false>(kst, xb, qw, my_rlut, nlive, m_lo, m_hi, c_hi, ones, tig, acc);
            if (nlive > 32)
                tile_compute<W, NB, false>(kst + 32 * W, xb + 32 * W, qw, my_rlut, nlive - 32, m_lo, m_hi, c_hi, ones, tig, acc);
        }
        nlive -= kTileKeys;
        kst = (tile % STAGES == STAGES - 1) ? ring : kst + TILE_WORDS;
    }
    cp_async_wait<0>();
    __syncwarp();  // the ring is free: the epilogue transposes through it

    // ---- undo the scales, transpose through shared memory, write the output row or a partial record -------
    // row gid of a channel block read bit gid of the half-word: an fp16 subnormal 2^(gid - 24);
    // row gid + 8 read bit b = gid + 8: 2^(b - 24) for b < 10, 2^(2^(b - 10) - 15) for b = 10..14, +-2 for b = 15
    const float f_lo = __uint_as_float(static_cast<uint32_t>(127 + 24 - gid) << 23);
    const int b_hi = gid + 8;
    const int e_hi = b_hi < 10 ? b_hi - 24 : (1 << (b_hi - 10)) - 15;
    const float f_hi = __uint_as_float(static_cast<uint32_t>(127 - e_hi) << 23);
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
        c0 *= f_lo; c1 *= f_lo;
        if (gid == 7) {  // sum of w * (2 - 4 bit) = 2 total - 4 sum
            c2 = (2.0f * tot0 - c2) * 0.25f;
            c3 = (2.0f * tot1 - c3) * 0.25f;
        } else {
            c2 *= f_hi; c3 *= f_hi;
        }
        ep[(2 * tig) * ES + 16 * jb + gid] = c0;
        ep[(2 * tig + 1) * ES + 16 * jb + gid] = c1;
        ep[(2 * tig) * ES + 16 * jb + 8 + gid] = c2;
        ep[(2 * tig + 1) * ES + 16 * jb + 8 + gid] = c3;
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
    if (n_units == 1) {
        if (hh < nh) {
            const float tot = ep[kAttnHeads * ES + hh];
            const float inv = tot > 0.0f ? 1.0f / tot : 0.0f;
            const int64_t idx = t * p.so_t + row * p.so_n + (h0 + hh) * p.so_h + tig * QC;
            if (p.out_dtype == SPK_F32) store_channels<QC>(static_cast<float*>(p.out) + idx, src, inv, sp.out_vec);
            else if (p.out_dtype == SPK_BF16) store_channels<QC>(static_cast<__nv_bfloat16*>(p.out) + idx, src, inv, sp.out_vec);
            else store_channels<QC>(static_cast<__half*>(p.out) + idx, src, inv, sp.out_vec);
        }
    } else {
        float* rec = p.ws + ((static_cast<int64_t>(row) * sp.gt + gt) * sp.max_units + unit) * sp.rec;
        store_channels<QC>(rec + hh * D + tig * QC, src, 1.0f, true);
        if (lane < kAttnHeads) rec[kAttnHeads * D + lane] = ep[kAttnHeads * ES + lane];
    }
}

// Sums the partial records of one (sequence, KV head, pass, timestep) in unit order and divides.  Rows of a
// single unit were written by the main kernel and are skipped.
__global__ void __launch_bounds__(128)
attn_stream_combine_kernel(const AttnParams p, const StreamParams sp, int D) {
    const int64_t item = blockIdx.x;  // row * gt_count + gt
    const int gt = static_cast<int>(item % sp.gt);
    const int64_t row = item / sp.gt;
    const int n_units = units_of(clamp_len(__ldg(p.lens + row), p.max_keys), sp.unit_log2);
    if (n_units <= 1) return;
    const int t = gt % p.T;
    const int gp = gt / p.T;
    const int g = gp / p.passes;
    const int pass = gp - g * p.passes;
    const int h0 = g * p.n_rep + pass * kAttnHeads;
    const int nh = min(kAttnHeads, p.n_rep - pass * kAttnHeads);
    // the records are complete once the main kernel's grid has finished and flushed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float* base = p.ws + item * sp.max_units * sp.rec;
    for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
        const int hh = idx / D;
        const int d = idx - hh * D;
        float a = 0.0f, l = 0.0f;
        for (int u = 0; u < n_units; ++u) {
            a += base[u * sp.rec + hh * D + d];
            l += base[u * sp.rec + kAttnHeads * D + hh];
        }
        const float v = l > 0.0f ? a / l : 0.0f;
        const int64_t o = t * p.so_t + row * p.so_n + (h0 + hh) * p.so_h + d;
        if (p.out_dtype == SPK_F32) static_cast<float*>(p.out)[o] = v;
        else if (p.out_dtype == SPK_BF16) static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
        else static_cast<__half*>(p.out)[o] = __float2half_rn(v);
    }
}

static inline int log2_exact(int x) {
    if (x < 1 || (x & (x - 1)) != 0) return -1;
    int l = 0;
    while ((1 << l) < x) ++l;
    return l;
}

template <int W, int NB>
int launch_stream(const AttnParams& p, const StreamParams& sp, int64_t ctas, cudaStream_t stream) {
    if (sp.dense) attn_stream_kernel<W, NB, true><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p, sp);
    else attn_stream_kernel<W, NB, false><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p, sp);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

}  // namespace

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
    // Largest unit that still gives every resident warp about two units when rows average half the table;
    // a unit's block-table entries must fit their staging (kTblMax) and a row at most 256 units.
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
    pl.rec_floats = static_cast<int64_t>(kAttnHeads) * head_dim + 8;
    pl.ws_bytes = max_units > 1 ? n_seqs * gt * max_units * pl.rec_floats * static_cast<int64_t>(sizeof(float)) : 0;
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

int spk_attn_stream_launch(const AttnParams& p, const StreamPlan& plan, int head_dim, cudaStream_t stream) {
    StreamParams sp;
    sp.unit_log2 = log2_exact(plan.unit_keys);
    sp.max_units = plan.max_units;
    sp.gt = p.T * p.Hkv * plan.passes;
    sp.dense = p.n_seqs <= kDenseRows;
    sp.rec = plan.rec_floats;
    const int esize = p.out_dtype == SPK_F32 ? 4 : 2;
    const int per = 16 / esize;
    sp.out_vec = reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && p.so_t % per == 0 && p.so_n % per == 0 && p.so_h % per == 0;
    // worst case of the enumeration: every row of max_units units (the surplus warps leave at once)
    const int64_t workers = p.n_seqs * plan.max_units * sp.gt;
    const int64_t ctas = (workers + kWarps - 1) / kWarps;
    if (ctas > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
    const bool wide = p.out_dtype == SPK_F32;  // fp32 output: {hi, lo} weights
    int rc;
    if (head_dim == 64) rc = wide ? launch_stream<2, 2>(p, sp, ctas, stream) : launch_stream<2, 1>(p, sp, ctas, stream);
    else rc = wide ? launch_stream<4, 2>(p, sp, ctas, stream) : launch_stream<4, 1>(p, sp, ctas, stream);
    if (rc != SPK_OK) return rc;
    if (plan.max_units > 1) {
        // Launched with programmatic stream serialisation: its CTAs may be placed while the main kernel still
        // runs (the launch latency overlaps), and each waits for the main grid before it reads a record.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(p.n_seqs * sp.gt));
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (p.n_seqs * sp.gt > 0x7fffffffLL) return SPK_ERR_TOO_LARGE;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, attn_stream_combine_kernel, p, sp, head_dim);
        if (e != cudaSuccess) return spk_set_cuda_error(e);
        spk_count_launch();
    }
    return SPK_OK;
}
