// Declarations shared by the two forms of the paged popcount decode attention:
//   spk_attn.cu         general form (any page size >= 1, any strides, head_dim 32..128, hi/lo weights)
//   spk_attn_stream.cu  streaming form (pages of >= 16 contiguous rows, head_dim 64 or 128)
#pragma once

#include "spk_common.cuh"

struct AttnParams {
    const uint32_t* q; int64_t sq_t, sq_n, sq_h;
    const uint32_t* k; int64_t sk_t, sk_h; int sk_blk, sk_slot;  // page and slot strides fit 31 bits (host-checked)
    const uint32_t* v; int64_t sv_t, sv_h; int sv_blk, sv_slot;
    const int32_t* tables; int64_t sbt_n;
    const int32_t* lens;
    void* out; int out_dtype; int64_t so_t, so_n, so_h;
    int T; int64_t n_seqs; int Hq, Hkv, n_rep, passes;
    int bs_log2; int max_keys, num_blocks;  // max_keys = max_blocks * block_size, below 2^31 (host-checked)
    float scale;
    float* ws; int splits; int granule;  // granule: keys per CTA step = 32 x warps per CTA (general form)
    int longest_first;  // rank rows by length in-kernel (only worth its dependent load when CTAs outnumber the slots)
    uint32_t* status;
    int overlap;  // the caller allows this launch to overlap the previous one on the stream (see spk_attn_overlap_next_call)
    int64_t items;
};

// Query heads served per pass over K and V: the eight columns of the MMA tile.
constexpr int kAttnHeads = 8;

// How the streaming form cuts the batch (see spk_attn_stream.cu).
struct StreamPlan {
    bool ok;            // the shape is one the streaming form handles
    bool dense;         // range form: the warps of the grid share one list of 32-key steps in equal parts
    bool cut;           // range form: some item may be cut between warps (records and a combine pass exist)
    int short_steps;    // range form: items of at most this many 32-key steps are never cut
    int64_t workers;    // range form: warps sharing the list
    int unit_keys;      // unit form: keys per unit (512, 1024 or 2048)
    int max_units;      // unit form: units of the longest possible row
    int passes;         // passes per KV head (eight query heads each)
    int64_t rec_floats; // floats per partial record: 8 * head_dim sums + 8 weight totals
    int64_t ws_bytes;   // partial records; 0 when nothing can be cut
};

// Form picked by spk_attn_select_form (SPK_ATTN_FORM_*).
int spk_attn_selected_form();

StreamPlan spk_attn_stream_plan(int T, int64_t n_seqs, int Hq, int Hkv, int head_dim, int block_size,
                                int64_t max_blocks);

// True when the layout allows the streaming form: rows of a page contiguous and 16-byte aligned.
bool spk_attn_stream_layout_ok(const AttnParams& p, int head_dim);

// Launches the streaming form (and its combine pass when rows are cut).  p.ws must hold plan.ws_bytes.
int spk_attn_stream_launch(const AttnParams& p, const StreamPlan& plan, int head_dim, cudaStream_t stream);
