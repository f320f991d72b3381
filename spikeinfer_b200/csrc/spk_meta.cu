// On-GPU continuous-batching metadata for decode steps.
//
// The reference rebuilds input ids, positions, the slot mapping, padded block tables and
// sequence lengths as Python lists on the host every step and ships them with five to seven
// host-to-device copies (spikeinfer/engine/model_runner.py:66-138), then copies them again into
// the static buffers of the captured graph (:275-287).  Here the same state lives on the device
// and one single-block kernel advances it, so a decode step needs no host-built tensor at all
// and the kernel can sit at the head of the captured graph.
//
// Allocation order mirrors BlockManager (spikeinfer/engine/block_manager.py:29,50-66): the free
// list is a stack handed out from its tail, rows are served in row order, a finished row returns
// its blocks in table order.
#include "spk_common.cuh"

namespace {

constexpr int kMaxRows = 1024;

__global__ void meta_init_kernel(int32_t* free_list, int32_t* free_count, int32_t num_alloc,
                                 int32_t* active, int32_t* seq_lens, int64_t* positions,
                                 int64_t* slot_mapping, int32_t* tables, int64_t* input_ids,
                                 int32_t max_rows, int32_t max_blocks, int32_t pad_block,
                                 int32_t block_size) {
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = tid; i < num_alloc; i += stride) free_list[i] = num_alloc - 1 - static_cast<int32_t>(i);
    for (int64_t i = tid; i < static_cast<int64_t>(max_rows) * max_blocks; i += stride) tables[i] = pad_block;
    for (int64_t i = tid; i < max_rows; i += stride) {
        active[i] = 0;
        seq_lens[i] = 1;
        positions[i] = 0;
        slot_mapping[i] = static_cast<int64_t>(pad_block) * block_size;
        input_ids[i] = 0;
    }
    if (tid == 0) *free_count = num_alloc;
}

// One block, one thread per row.
__global__ void __launch_bounds__(kMaxRows)
meta_advance_kernel(int32_t* free_list, int32_t* free_count, const int32_t* active,
                    int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping, int32_t* tables,
                    int64_t* input_ids, const int64_t* next_tokens, int32_t max_rows,
                    int32_t max_blocks, int32_t pad_block, int32_t block_size, uint32_t* status) {
    __shared__ int warp_tot[32];
    const int row = threadIdx.x;
    const int lane = row & 31;
    const int wid = row >> 5;
    const bool in_range = row < max_rows;
    const bool act = in_range && active[row] != 0;
    int pos = 0;
    bool need = false;
    bool full = false;
    if (act) {
        pos = seq_lens[row];
        if (pos < 0) pos = 0;
        full = pos / block_size >= max_blocks;
        need = !full && (pos % block_size == 0);
        if (full) spk_flag(status, SPK_STATUS_TABLE_FULL);
    }
    // exclusive prefix count of `need` in row order
    const unsigned ballot = __ballot_sync(0xffffffffu, need);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[wid] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
    const int n_warps = (blockDim.x + 31) >> 5;
    for (int w = 0; w < n_warps; ++w) {
        const int c = warp_tot[w];
        if (w < wid) before += c;
        total += c;
    }
    const int rank = before + in_warp;
    const int fc = *free_count;
    __syncthreads();  // every thread has read free_count before it changes

    if (in_range) {
        if (act && !full) {
            bool ok = true;
            if (need) {
                if (rank < fc) {
                    tables[static_cast<int64_t>(row) * max_blocks + pos / block_size] = free_list[fc - 1 - rank];
                } else {
                    spk_flag(status, SPK_STATUS_POOL_EXHAUSTED);
                    ok = false;
                }
            }
            if (ok) {
                const int32_t blk = tables[static_cast<int64_t>(row) * max_blocks + pos / block_size];
                positions[row] = pos;
                slot_mapping[row] = static_cast<int64_t>(blk) * block_size + pos % block_size;
                seq_lens[row] = pos + 1;
            } else {
                slot_mapping[row] = static_cast<int64_t>(pad_block) * block_size;
            }
            if (next_tokens != nullptr) input_ids[row] = next_tokens[row];
        } else if (!act) {
            seq_lens[row] = 1;
            positions[row] = 0;
            slot_mapping[row] = static_cast<int64_t>(pad_block) * block_size;
        } else {
            slot_mapping[row] = static_cast<int64_t>(pad_block) * block_size;
        }
    }
    if (threadIdx.x == 0) *free_count = fc - min(total, fc);
}

__global__ void meta_take_kernel(int32_t* free_list, int32_t* free_count, int32_t count,
                                 int32_t* dst, uint32_t* status) {
    const int fc = *free_count;
    __syncthreads();
    if (count > fc) {
        if (threadIdx.x == 0) spk_flag(status, SPK_STATUS_POOL_EXHAUSTED);
        return;
    }
    for (int i = threadIdx.x; i < count; i += blockDim.x) dst[i] = free_list[fc - 1 - i];
    if (threadIdx.x == 0) *free_count = fc - count;
}

__global__ void meta_admit_kernel(int32_t row, const int32_t* src_table, int32_t seq_len,
                                  int64_t last_token, int32_t* active, int32_t* seq_lens,
                                  int64_t* positions, int64_t* slot_mapping, int32_t* tables,
                                  int64_t* input_ids, int64_t* next_tokens, int32_t max_blocks,
                                  int32_t pad_block, int32_t block_size, uint32_t* status) {
    // a row that still holds a sequence keeps it: overwriting its table would leak its blocks
    const bool busy = active[row] != 0;
    __syncthreads();
    if (busy) {
        if (threadIdx.x == 0) spk_flag(status, SPK_STATUS_ROW_BUSY);
        return;
    }
    const int nb = (seq_len + block_size - 1) / block_size;
    for (int i = threadIdx.x; i < max_blocks; i += blockDim.x)
        tables[static_cast<int64_t>(row) * max_blocks + i] = i < nb ? src_table[i] : pad_block;
    if (threadIdx.x == 0) {
        active[row] = 1;
        seq_lens[row] = seq_len;
        positions[row] = seq_len > 0 ? seq_len - 1 : 0;
        slot_mapping[row] = static_cast<int64_t>(pad_block) * block_size;
        input_ids[row] = last_token;
        if (next_tokens != nullptr) next_tokens[row] = last_token;
    }
}

__global__ void meta_release_kernel(int32_t row, int32_t* free_list, int32_t* free_count,
                                    int32_t* active, int32_t* seq_lens, int64_t* positions,
                                    int64_t* slot_mapping, int32_t* tables, int32_t max_blocks,
                                    int32_t pad_block, int32_t block_size, int32_t num_alloc,
                                    uint32_t* status) {
    const int fc = *free_count;
    const int len = active[row] != 0 ? seq_lens[row] : 0;
    int nb = (len + block_size - 1) / block_size;
    if (nb > max_blocks) nb = max_blocks;
    __syncthreads();
    if (fc < 0 || fc + nb > num_alloc) {
        // more blocks coming back than ever left the list (the count was not kept in step with the
        // tables): nothing is pushed, the row is still retired
        if (threadIdx.x == 0) spk_flag(status, SPK_STATUS_FREE_LIST_OVERFLOW);
        nb = 0;
    }
    for (int i = threadIdx.x; i < max_blocks; i += blockDim.x) {
        int32_t* e = tables + static_cast<int64_t>(row) * max_blocks + i;
        if (i < nb) free_list[fc + i] = *e;
        *e = pad_block;
    }
    if (threadIdx.x == 0) {
        *free_count = fc + nb;
        active[row] = 0;
        seq_lens[row] = 1;
        positions[row] = 0;
        slot_mapping[row] = static_cast<int64_t>(pad_block) * block_size;
    }
}

}  // namespace

extern "C" int spk_meta_init(int32_t* free_list, int32_t* free_count, int32_t num_alloc_blocks,
                             int32_t* active, int32_t* seq_lens, int64_t* positions,
                             int64_t* slot_mapping, int32_t* block_tables, int64_t* input_ids,
                             int32_t max_rows, int32_t max_blocks, int32_t pad_block,
                             int32_t block_size, void* stream) {
    if (num_alloc_blocks < 0 || max_rows < 1 || max_rows > kMaxRows || max_blocks < 1 || block_size < 1)
        return SPK_ERR_BAD_SHAPE;
    if (free_list == nullptr || free_count == nullptr || active == nullptr || seq_lens == nullptr ||
        positions == nullptr || slot_mapping == nullptr || block_tables == nullptr || input_ids == nullptr)
        return SPK_ERR_NULL_POINTER;
    meta_init_kernel<<<148, 256, 0, spk_stream(stream)>>>(free_list, free_count, num_alloc_blocks, active,
                                                          seq_lens, positions, slot_mapping, block_tables,
                                                          input_ids, max_rows, max_blocks, pad_block,
                                                          block_size);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_meta_advance(int32_t* free_list, int32_t* free_count, const int32_t* active,
                                int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping,
                                int32_t* block_tables, int64_t* input_ids, const int64_t* next_tokens,
                                int32_t max_rows, int32_t max_blocks, int32_t pad_block,
                                int32_t block_size, uint32_t* status, void* stream) {
    SpkRange nvtx_range("spk_meta_advance");
    if (max_rows < 1 || max_rows > kMaxRows || max_blocks < 1 || block_size < 1) return SPK_ERR_BAD_SHAPE;
    if (free_list == nullptr || free_count == nullptr || active == nullptr || seq_lens == nullptr ||
        positions == nullptr || slot_mapping == nullptr || block_tables == nullptr || input_ids == nullptr)
        return SPK_ERR_NULL_POINTER;
    const int threads = ((max_rows + 31) / 32) * 32;
    meta_advance_kernel<<<1, threads, 0, spk_stream(stream)>>>(free_list, free_count, active, seq_lens,
                                                               positions, slot_mapping, block_tables,
                                                               input_ids, next_tokens, max_rows, max_blocks,
                                                               pad_block, block_size, status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_meta_take(int32_t* free_list, int32_t* free_count, int32_t count, int32_t* dst_table,
                             uint32_t* status, void* stream) {
    if (count < 0) return SPK_ERR_BAD_SHAPE;
    if (count == 0) return SPK_OK;
    if (free_list == nullptr || free_count == nullptr || dst_table == nullptr) return SPK_ERR_NULL_POINTER;
    meta_take_kernel<<<1, 256, 0, spk_stream(stream)>>>(free_list, free_count, count, dst_table, status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_meta_admit(int32_t row, const int32_t* src_table, int32_t seq_len, int64_t last_token,
                              int32_t* active, int32_t* seq_lens, int64_t* positions,
                              int64_t* slot_mapping, int32_t* block_tables, int64_t* input_ids,
                              int64_t* next_tokens, int32_t max_rows, int32_t max_blocks,
                              int32_t pad_block, int32_t block_size, uint32_t* status, void* stream) {
    if (row < 0 || row >= max_rows || max_blocks < 1 || block_size < 1 || seq_len < 0) return SPK_ERR_BAD_SHAPE;
    if ((static_cast<int64_t>(seq_len) + block_size - 1) / block_size > max_blocks) return SPK_ERR_TOO_LARGE;
    if (src_table == nullptr || active == nullptr || seq_lens == nullptr || positions == nullptr ||
        slot_mapping == nullptr || block_tables == nullptr || input_ids == nullptr)
        return SPK_ERR_NULL_POINTER;
    meta_admit_kernel<<<1, 256, 0, spk_stream(stream)>>>(row, src_table, seq_len, last_token, active, seq_lens,
                                                         positions, slot_mapping, block_tables, input_ids,
                                                         next_tokens, max_blocks, pad_block, block_size, status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}

extern "C" int spk_meta_release(int32_t row, int32_t* free_list, int32_t* free_count, int32_t* active,
                                int32_t* seq_lens, int64_t* positions, int64_t* slot_mapping,
                                int32_t* block_tables, int32_t max_rows, int32_t max_blocks,
                                int32_t pad_block, int32_t block_size, int32_t num_alloc_blocks,
                                uint32_t* status, void* stream) {
    if (row < 0 || row >= max_rows || max_blocks < 1 || block_size < 1 || num_alloc_blocks < 0) return SPK_ERR_BAD_SHAPE;
    if (free_list == nullptr || free_count == nullptr || active == nullptr || seq_lens == nullptr ||
        positions == nullptr || slot_mapping == nullptr || block_tables == nullptr)
        return SPK_ERR_NULL_POINTER;
    meta_release_kernel<<<1, 256, 0, spk_stream(stream)>>>(row, free_list, free_count, active, seq_lens,
                                                           positions, slot_mapping, block_tables, max_blocks,
                                                           pad_block, block_size, num_alloc_blocks, status);
    SPK_CHECK_LAUNCH();
    return SPK_OK;
}
