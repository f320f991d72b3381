/*
 * spikeinfer_b200 -- C ABI of the sm_100a spiking-decode kernels.
 *
 * Every entry point takes plain device pointers, element strides and sizes; no
 * torch types cross this boundary.  All launches are asynchronous on the CUDA
 * stream passed as `stream` (a cudaStream_t cast to void*, NULL = legacy default
 * stream) and none of them synchronises the device, allocates device memory or
 * retains a pointer after returning.  The operator entry points (spk_pack .. spk_meta_*)
 * may therefore be recorded in a CUDA graph; spk_attn_decode_static has rules of its own.
 *
 * Return value: 0 on success, a negative SPK_ERR_* code when the arguments are
 * rejected on the host (nothing was launched), SPK_ERR_CUDA when the launch
 * itself failed (spk_last_cuda_error() holds the cudaError_t).
 *
 * Device-detected anomalies (a block-table entry or slot outside the pool, a
 * sequence length outside [1, max_blocks * block_size], an exhausted free list)
 * never trap: the offending access is skipped and a bit is OR-ed into the
 * caller-provided `status` word (device memory, may be NULL).  The host reads
 * the word whenever it is convenient.
 *
 * "Reference" below is HzAybars/Spikeinfer v0.3.0; file:line citations are paths
 * inside that project.
 */
#ifndef SPIKEINFER_B200_H
#define SPIKEINFER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- element types -------------------------------------------------------- */
enum {
    SPK_F32 = 0,
    SPK_BF16 = 1,
    SPK_F16 = 2,
    SPK_U8 = 3,
    SPK_I32 = 4
};

/* ---- LIF reset rules ------------------------------------------------------ */
enum {
    /* r_t = H(U_{t-1}-theta); U_t = clamp(beta,0,1)*U_{t-1} + I_t - r_t*theta; S_t = H(U_t-theta).
     * The only rule the reference implements (spikeinfer/kernels/lif_triton.py:13-15). */
    SPK_RESET_SUBTRACT_DELAYED = 0,
    /* U_t = clamp(beta,0,1)*U_{t-1} + I_t; S_t = H(U_t-theta); U_t <- 0 where S_t = 1.
     * Not in the reference; checked only against this library's own CPU restatement. */
    SPK_RESET_HARD_ZERO = 1
};

/* ---- host-side error codes ------------------------------------------------ */
enum {
    SPK_OK = 0,
    SPK_ERR_BAD_DTYPE = -1,
    SPK_ERR_BAD_SHAPE = -2,
    SPK_ERR_BAD_STRIDE = -3,
    SPK_ERR_NULL_POINTER = -4,
    SPK_ERR_WORKSPACE_TOO_SMALL = -5,
    SPK_ERR_UNSUPPORTED = -6,
    SPK_ERR_TOO_LARGE = -7,
    SPK_ERR_STATIC_SCRATCH_TOO_SMALL = -8,
    SPK_ERR_CUDA = -100
};

/* ---- bits of the device status word --------------------------------------- */
enum {
    SPK_STATUS_BAD_BLOCK = 1u << 0,     /* block-table entry outside [0, num_blocks)        */
    SPK_STATUS_BAD_SEQ_LEN = 1u << 1,   /* seq_len < 1 or > max_blocks * block_size         */
    SPK_STATUS_BAD_SLOT = 1u << 2,      /* slot_mapping entry outside [0, num_slots)        */
    SPK_STATUS_POOL_EXHAUSTED = 1u << 3,/* metadata builder ran out of free blocks          */
    SPK_STATUS_TABLE_FULL = 1u << 4,    /* a row needs more than max_blocks blocks          */
    SPK_STATUS_FREE_LIST_OVERFLOW = 1u << 5, /* a release would push past the list's capacity    */
    SPK_STATUS_ROW_BUSY = 1u << 6,      /* admit into a row that still holds a sequence      */
    SPK_STATUS_DEVICE_WAIT_EXPIRED = 1u << 7 /* a kernel gave up waiting for its own tensor-core work;
                                            the affected rows of the output are zero           */
};

/* Library version, (major << 16) | (minor << 8) | patch. */
int spk_version(void);
/* cudaError_t of the most recent failed launch in this thread (0 if none). */
int spk_last_cuda_error(void);
/* Static description of an SPK_ERR_* code. */
const char* spk_error_string(int code);
/* Kernels this library has launched (or recorded into a CUDA graph being captured) in this process.
 * No counterpart in the reference; used to report launch counts honestly. */
int64_t spk_launch_count(void);
/* 1 when the entry points that launch the decode path's kernels (attention, LIF, metadata advance, norm,
 * argmax) wrap their launches in NVTX ranges named after themselves, else 0.  Decided once per process from
 * the environment: SPK_NVTX set to anything but "" or "0".  No counterpart in the reference. */
int spk_nvtx_enabled(void);

/* ---------------------------------------------------------------------------
 * Bit packing.  Replaces pack_spikes / _pack_kernel and unpack_spikes
 * (spikeinfer/kernels/packing.py:84-133, :57-81, :136-152).
 *
 * x is a strided [d0, .., d_{ndim-1}, C] array (ndim <= 6 leading dims, sizes and
 * element strides given as host arrays; the channel axis has stride 1).  Anything
 * != 0 packs as 1.  Bit i of word w holds channel 32*w + i; the tail of the last
 * word is zero.  out is contiguous int32 [rows, ceil(C/32)].
 * ------------------------------------------------------------------------- */
int spk_pack(const void* x, int x_dtype, int ndim, const int64_t* sizes, const int64_t* strides,
             int64_t channels, int32_t* out, void* stream);

/* words: contiguous int32 [rows, ceil(C/32)] -> out: contiguous [rows, C] of 0/1 in out_dtype. */
int spk_unpack(const int32_t* words, int64_t rows, int64_t channels, void* out, int out_dtype,
               void* stream);

/* ---------------------------------------------------------------------------
 * Fused T-step LIF recurrence, dense spike output.  Replaces lif_multistep /
 * _lif_multistep_fwd (spikeinfer/kernels/lif_triton.py:141-233, :48-105).
 *
 * x is a strided [T, m0, .., m_{n_mid-1}, N] array (n_mid <= 6; channel stride 1).
 * beta / threshold are fp32 [N]; beta is clamped to [0,1] inside the kernel.
 * mem0 (optional) and mem_out (optional) are contiguous fp32 [M, N], M = prod(m_i).
 * spikes is contiguous [T, M, N] of 0/1 in spike_dtype.  Every operation is an
 * individually rounded fp32 mul/add/sub in the order ((beta*u) + I) - (r*theta);
 * the spike predicate is (u - theta) > 0.
 * ------------------------------------------------------------------------- */
int spk_lif(const void* x, int x_dtype, int T, int64_t stride_t, int n_mid,
            const int64_t* mid_sizes, const int64_t* mid_strides, int64_t N, const float* beta,
            const float* threshold, const float* mem0, void* spikes, int spike_dtype,
            float* mem_out, int reset_mode, void* stream);

/* ---------------------------------------------------------------------------
 * Fused LIF + bit-pack + slot-mapped scatter.  One launch covers up to
 * SPK_MAX_LIF_SITES neuron sites (e.g. the q, k and v sites of one layer).
 * Replaces, per site, lif_multistep (lif_triton.py:141) followed by pack_spikes
 * (packing.py:84) and, for k/v, cache.index_copy_(2, slot_mapping, packed)
 * (spikeinfer/attention.py:138-139); for q it also absorbs the permute + pack of
 * attention.py:146-148.
 *
 * Site input: x[t, tok, h, c] at x + t*sx_t + tok*sx_tok + h*sx_h + c, c < N.
 * Packed output word (t, tok, h, w) goes to
 *     packed + t*so_t + row*so_tok + h*so_h + w,
 * row = slot_mapping[tok] when slot_mapping != NULL (rows outside [0, num_rows)
 * are skipped and flagged), else row = tok.  dense (optional) receives the 0/1
 * spikes at dense + t*sd_t + tok*sd_tok + h*sd_h + c in dense_dtype.  mem0 /
 * mem_out (optional) are contiguous fp32 [n_tok, H, N].  The rope_* and mul/gated fields need
 * N % 32 == 0 and 16-byte-aligned rows (SPK_ERR_UNSUPPORTED otherwise).
 * ------------------------------------------------------------------------- */
#define SPK_MAX_LIF_SITES 4

typedef struct spk_lif_site {
    const void* x;
    int32_t x_dtype;
    int32_t H;
    int64_t N;
    int64_t sx_t, sx_tok, sx_h;
    const float* beta;
    const float* threshold;
    const float* mem0;
    float* mem_out;
    int32_t* packed;
    int64_t so_t, so_tok, so_h;
    const int64_t* slot_mapping;
    int64_t num_rows;
    void* dense;
    int32_t dense_dtype;
    int32_t _pad;
    int64_t sd_t, sd_tok, sd_h;
    /* Optional rotary embedding applied to the currents before the neuron (q and k sites):
     * cos/sin [n_tok, N] in the dtype of x, row stride s_rope_tok.  Arithmetic is
     * (x * cos) + (rotate_half(x) * sin) with every operation rounded to that dtype, as
     * _apply_rope_t does (spikeinfer/modeling_fast.py:89-99).  NULL = none. */
    const void* rope_cos;
    const void* rope_sin;
    int64_t s_rope_tok;
    /* Optional gated product (the MLP's gate_spk * up_proj(x), modeling_fast.py:190):
     * gated[t, tok, h, c] = spike ? mul[t, tok, h, c] : 0, both in the dtype of x.  NULL = none. */
    const void* mul;
    int64_t sm_t, sm_tok, sm_h;
    void* gated;
    int64_t sg_t, sg_tok, sg_h;
} spk_lif_site;

int spk_lif_pack_scatter(const spk_lif_site* sites, int n_sites, int T, int64_t n_tok,
                         int reset_mode, uint32_t* status, void* stream);

/* ---------------------------------------------------------------------------
 * Residual add + RMSNorm.  Replaces `h = h + delta` and the Qwen2RMSNorm call of a decoder layer
 * (spikeinfer/modeling_fast.py:206-211, :319).  h [rows, hidden] (contiguous, updated in place when
 * delta != NULL: h <- round(h + delta)), out [rows, hidden] = weight * (h * rsqrt(mean(h^2) + eps))
 * with the variance in fp32 and the normalised value rounded to the dtype before the weight, as
 * Qwen2RMSNorm does.  out may not alias h.
 * ------------------------------------------------------------------------- */
int spk_add_rmsnorm(void* h, const void* delta, const void* weight, float eps, void* out, int64_t rows,
                    int64_t hidden, int dtype, void* stream);

/* ---------------------------------------------------------------------------
 * Greedy sampling: out[r] = argmax over x[r, 0..cols) with torch.argmax's rules (first index of the
 * largest value; NaN is larger than everything).  Replaces `logits.argmax(dim=-1)` of the sampler
 * (spikeinfer/engine/sampler.py:63-81) so that the choice stays on the device, inside the captured
 * decode step.  x [rows, cols] in F32/BF16/F16 with row stride row_stride (elements); out int64 [rows];
 * workspace of spk_argmax_workspace_bytes(rows) bytes, 8-byte aligned.  rows <= 65535.
 * ------------------------------------------------------------------------- */
int64_t spk_argmax_workspace_bytes(int64_t rows);
int spk_argmax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int64_t* out,
               void* workspace, int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * Paged popcount decode attention.  Replaces paged_spike_attn_decode /
 * _paged_spike_attn_decode_kernel (spikeinfer/kernels/spike_attention.py:153-221,
 * :67-150) and the SWAR _popc (:52-65).
 *
 * q        int32 [T, n_seqs, H_q, W]      strides sq_t, sq_n, sq_h (word stride 1)
 * k, v     int32 pools addressed as base + t*s_t + kv_head*s_h + block*s_blk
 *          + slot_in_block*s_slot + w.  The reference layout [T, H_kv, num_slots, W]
 *          (spikeinfer/engine/spike_cache.py:51) is s_slot = W, s_blk = block_size*W.
 * block_tables int32 [n_seqs, max_blocks] (row stride sbt_n), seq_lens int32 [n_seqs]
 *          (length including the token being decoded; its K/V must already be written).
 * out      [T, n_seqs, H_q, head_dim] in out_dtype (F32/BF16/F16), strides so_t, so_n,
 *          so_h (channel stride 1) -- may be a view of a larger buffer.
 *
 * scores are exact integers popc(q & k); the weighted sum p.v runs on the tensor cores with
 * fp32 accumulation.  For F32 output the softmax weights are carried as pairs of fp16 numbers
 * (22 significant bits; within 1e-6 of a float64 evaluation, relative to the largest output);
 * for BF16/F16 output one fp16 weight is used in numerator and denominator alike (within 1e-3
 * before the rounding to the output type).  K and V are read once per KV head, shared by the
 * H_q/H_kv query heads of the group.  Rows longer than 256 keys may be cut into key ranges (equal
 * shares of the call's 32-key steps per warp when pages are contiguous 16-byte aligned rows at
 * head_dim 64/128, else ranges per row) whose partial sums live in `workspace`
 * (size from spk_attn_decode_workspace_bytes with the same arguments; may be NULL when that
 * returns 0).  head_dim must be a multiple of 32, <= 128; block_size a power of two, >= 1;
 * 0 <= scale and scale * head_dim <= 24 (head_dim^-0.5, the reference's scale, always is), else
 * SPK_ERR_UNSUPPORTED; max_blocks * block_size + 800, num_blocks and the block/slot strides
 * must fit 31 bits, else SPK_ERR_TOO_LARGE.
 * ------------------------------------------------------------------------- */
int64_t spk_attn_decode_workspace_bytes(int T, int64_t n_seqs, int num_q_heads, int num_kv_heads,
                                        int head_dim, int block_size, int64_t max_blocks);

int spk_attn_decode(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                    const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                    const int32_t* v, int64_t sv_t, int64_t sv_h, int64_t sv_blk, int64_t sv_slot,
                    const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                    void* out, int out_dtype, int64_t so_t, int64_t so_n, int64_t so_h,
                    int T, int64_t n_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                    int block_size, int64_t max_blocks, int64_t num_blocks, float scale,
                    void* workspace, int64_t workspace_bytes, uint32_t* status, void* stream);

/* Lets the NEXT spk_attn_decode / spk_attn_decode_static call of this host thread overlap the launch that
 * precedes it on its stream (programmatic dependent launch): the attention grid is placed while that launch
 * still runs, reads seq_lens and block_tables, and waits for the launch to finish before it touches q, the
 * pools, the workspace or `out`.  The caller vouches that seq_lens and block_tables were complete before the
 * preceding launch BEGAN (in a decode step they are written at the head of the step, and the preceding launch is
 * spk_lif_pack_scatter, which produces q and the newest K/V rows).  One-shot: it applies to one call and is
 * cleared by it, also when that call returns an error.  Results are the same with and without it.  Returns
 * SPK_OK.  No
 * counterpart in the reference. */
int spk_attn_overlap_next_call(void);

/* Which form of the attention kernel spk_attn_decode takes (no counterpart in the reference; it lets tests and
 * benchmarks run one form against another).  AUTO: the streaming mma.sync form where the layout allows it
 * (pages of contiguous, 16-byte aligned rows, head_dim 64 or 128), else the general form.  GENERAL: always the
 * general form.  TCGEN05: the tcgen05 / tensor-memory form where it applies (head_dim 64, BF16/F16 output, at most
 * 1024 sequences, scale * head_dim <= 16), else as AUTO.  Process-wide; returns SPK_ERR_UNSUPPORTED for other values. */
enum {
    SPK_ATTN_FORM_AUTO = 0,
    SPK_ATTN_FORM_GENERAL = 1,
    SPK_ATTN_FORM_TCGEN05 = 2
};
int spk_attn_select_form(int form);

/* spk_attn_decode for callers that cannot allocate (no counterpart in the reference).
 *
 * Same arguments and results as spk_attn_decode, minus the workspace: the partial sums of split
 * rows go to a fixed SPK_ATTN_STATIC_SCRATCH_BYTES array inside the library instead.  It exists for
 * processes that handed all free device memory to the page pool at start-up, and for hosts that
 * drive the library through an FFI with nothing but the pointers they were given: neither can
 * produce a workspace.  The cost is that every GPU that loads the library holds the array until
 * the process ends.
 *
 *  - No cudaMalloc / cudaFree and no other allocating call is made, here or on first use.
 *  - A problem whose spk_attn_decode_workspace_bytes() exceeds spk_attn_decode_static_capacity()
 *    is refused with SPK_ERR_STATIC_SCRATCH_TOO_SMALL and nothing is launched.  Tables of up to
 *    256 keys per sequence (max_blocks * block_size) need no scratch at all.  Beyond that the need
 *    grows with n_seqs * T * H_kv * max_blocks * block_size (two records of 8 * head_dim + 8 floats
 *    per warp that shares the work, up to 2368 warps): at T=4, 14/2
 *    heads, head_dim 64, 15 sequences of up to 4096 keys need 7.99 MB and fit, 16 such sequences
 *    (8.52 MB) do not.
 *  - The first call on each device, whatever its sizes (a problem that needs no scratch included),
 *    looks up the array's device address with that device current and remembers it; make that
 *    first call during start-up, before any stream capture begins.  Later calls only read the
 *    remembered address.
 *  - All calls on a device share the one array and it keeps whatever the last call wrote.  Nothing
 *    in it has to start at zero (each call writes every record it later reads), but two calls
 *    whose kernels overlap on the GPU, e.g. on different streams, race on it: one call at a time
 *    per device. */
#define SPK_ATTN_STATIC_SCRATCH_BYTES (8ll << 20)
int64_t spk_attn_decode_static_capacity(void);
int spk_attn_decode_static(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                           const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                           const int32_t* v, int64_t sv_t, int64_t sv_h, int64_t sv_blk, int64_t sv_slot,
                           const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                           void* out, int out_dtype, int64_t so_t, int64_t so_n, int64_t so_h,
                           int T, int64_t n_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                           int block_size, int64_t max_blocks, int64_t num_blocks, float scale,
                           uint32_t* status, void* stream);

/* Exact q.k scores, for checking: scores[t, n, h, j] = popc(q[t,n,h] & k[t, h/n_rep, key j])
 * for j < seq_lens[n], -1 for seq_lens[n] <= j < max_len.  scores is contiguous int32
 * [T, n_seqs, H_q, max_len].  The integer half of spike_attention.py:114-120. */
int spk_qk_scores(const int32_t* q, int64_t sq_t, int64_t sq_n, int64_t sq_h,
                  const int32_t* k, int64_t sk_t, int64_t sk_h, int64_t sk_blk, int64_t sk_slot,
                  const int32_t* block_tables, int64_t sbt_n, const int32_t* seq_lens,
                  int32_t* scores, int64_t max_len, int T, int64_t n_seqs, int num_q_heads,
                  int num_kv_heads, int head_dim, int block_size, int64_t max_blocks,
                  int64_t num_blocks, uint32_t* status, void* stream);

/* Dense read-back of one sequence for the prefill path.  Replaces gather_kv_unpacked
 * (spikeinfer/kernels/spike_attention.py:224-244): out[t, h, s, c] (contiguous
 * [T, H_kv, seq_len, head_dim] in out_dtype) = bit c of the word row at position s. */
int spk_gather_kv_unpacked(const int32_t* cache, int64_t s_t, int64_t s_h, int64_t s_blk,
                           int64_t s_slot, const int32_t* block_table, int64_t seq_len, int T,
                           int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
                           void* out, int out_dtype, uint32_t* status, void* stream);
/* The same for n_seqs sequences of equal length in one launch: block_tables int32 [n_seqs, >= ceil(seq_len / bs)]
 * with row stride sbt_n, out contiguous [n_seqs, T, H_kv, seq_len, head_dim].  Lets the prefill path read back all
 * chunks of one shape at once instead of one launch per sequence (the reference loops, spikeinfer/attention.py:161-178). */
int spk_gather_kv_unpacked_batch(const int32_t* cache, int64_t s_t, int64_t s_h, int64_t s_blk,
                                 int64_t s_slot, const int32_t* block_tables, int64_t sbt_n, int64_t n_seqs,
                                 int64_t seq_len, int T, int num_kv_heads, int head_dim, int block_size,
                                 int64_t num_blocks, void* out, int out_dtype, uint32_t* status, void* stream);

/* ---------------------------------------------------------------------------
 * On-GPU continuous-batching metadata for decode.  Replaces the decode half of
 * ModelRunner.prepare (spikeinfer/engine/model_runner.py:66-138), the five buffer
 * copies of CUDAGraphRunner.replay (:275-287) and mirrors BlockManager.allocate /
 * slot_mapping / free (spikeinfer/engine/block_manager.py:50-77).
 *
 * State, all in device memory and owned by the caller:
 *   free_list  int32 [num_alloc_blocks]  stack; entries [0, *free_count) are free and the
 *                                        next block handed out is free_list[*free_count-1]
 *   free_count int32 [1]
 *   active     int32 [max_rows]          1 = row holds a running sequence
 *   seq_lens   int32 [max_rows]          cached length (after advance: including the new token)
 *   positions  int64 [max_rows]
 *   slot_mapping int64 [max_rows]
 *   block_tables int32 [max_rows, max_blocks]
 *   input_ids  int64 [max_rows]
 * ------------------------------------------------------------------------- */

/* free_list <- [num_alloc_blocks-1 .. 0] (so blocks are handed out as 0,1,2,..., like
 * block_manager.py:29), *free_count <- num_alloc_blocks, every row inactive and pointed at the
 * pad block / pad slot with seq_len 1 (model_runner.py:234-248). */
int spk_meta_init(int32_t* free_list, int32_t* free_count, int32_t num_alloc_blocks,
                  int32_t* active, int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping,
                  int32_t* block_tables, int64_t* input_ids, int32_t max_rows, int32_t max_blocks,
                  int32_t pad_block, int32_t block_size, void* stream);

/* One decode step for every active row, in row order: position = seq_len; a row whose position
 * crosses a block boundary pops one block (row order = allocation order, as the scheduler's loop
 * over running sequences does); slot = table[pos / bs] * bs + pos % bs; seq_len += 1;
 * input_ids[row] = next_tokens[row] (skipped when next_tokens is NULL).  Inactive rows are left
 * at the pad slot with seq_len 1. */
int spk_meta_advance(int32_t* free_list, int32_t* free_count, const int32_t* active,
                     int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping,
                     int32_t* block_tables, int64_t* input_ids, const int64_t* next_tokens,
                     int32_t max_rows, int32_t max_blocks, int32_t pad_block, int32_t block_size,
                     uint32_t* status, void* stream);

/* Install a prefilled sequence in `row`: its first ceil(seq_len / bs) table entries are copied from
 * src_table (device int32), the rest of the row is the pad block; the blocks must have been removed
 * from the free list by spk_meta_take.  last_token, the token sampled after prefill, becomes
 * input_ids[row] and, when next_tokens != NULL, next_tokens[row], so that the following
 * spk_meta_advance feeds it to the model.  A row that is still active is left as it is and
 * SPK_STATUS_ROW_BUSY is set (overwriting it would leak its blocks). */
int spk_meta_admit(int32_t row, const int32_t* src_table, int32_t seq_len, int64_t last_token,
                   int32_t* active, int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping,
                   int32_t* block_tables, int64_t* input_ids, int64_t* next_tokens,
                   int32_t max_rows, int32_t max_blocks, int32_t pad_block, int32_t block_size,
                   uint32_t* status, void* stream);

/* Pop `count` blocks for a new sequence into dst_table[0..count) (allocation order = pop order). */
int spk_meta_take(int32_t* free_list, int32_t* free_count, int32_t count, int32_t* dst_table,
                  uint32_t* status, void* stream);

/* Finish `row`: push its ceil(seq_len / bs) blocks back in table order
 * (block_manager.py:63-66), reset the row to the pad state.  num_alloc_blocks is the capacity of
 * free_list: a push that would pass it is skipped and SPK_STATUS_FREE_LIST_OVERFLOW is set. */
int spk_meta_release(int32_t row, int32_t* free_list, int32_t* free_count, int32_t* active,
                     int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping,
                     int32_t* block_tables, int32_t max_rows, int32_t max_blocks,
                     int32_t pad_block, int32_t block_size, int32_t num_alloc_blocks,
                     uint32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPIKEINFER_B200_H */
