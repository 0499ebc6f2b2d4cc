// Row selection of the sparse decode kernels.  The reference passes flat physical token ids and reads
// them unchecked (kernels/dsa/naive_dsa.cu:13-59; page_size and total_kv_tokens are carried in DsaConfig
// and never used, kernels/dsa/naive_dsa.cuh:15-16).  Here an entry of the index list is resolved to a
// physical row or to "empty":
//   * entries at or beyond the query's valid length (valid_len, optional) are empty;
//   * negative entries (padding slots of a top-k list) are empty;
//   * with a block table the entry is a logical position of the query's sequence and is translated through
//     the sequence's page list (page = block_table[seq, pos / page_size]; a negative page is empty);
//   * rows outside [0, total_kv_tokens) are empty (when total_kv_tokens > 0).
// An empty entry contributes nothing: its score is -inf, its K/V rows are not read (the shared-memory rows
// are zero-filled), exactly as if it had been removed from the list.  A query whose entries are all empty
// gets a zero output row.
#pragma once

struct DsaIndex {
    const int* idx;           // [Q, S] physical row ids, or logical positions when block_table != NULL
    const int* block_table;   // [num_seqs, max_blocks] or NULL
    const int* seq_of_query;  // [Q] or NULL (query q reads sequence q)
    const int* valid_len;     // [Q] or NULL (all S entries count)
    int S, page, max_blocks, N;
};

__device__ __forceinline__ int dsa_resolve(const DsaIndex& ix, int q, int s) {
    if (ix.valid_len && s >= ix.valid_len[q]) return -1;
    int pos = ix.idx[(size_t)q * ix.S + s];
    if (pos < 0) return -1;
    if (ix.block_table) {
        const int seq = ix.seq_of_query ? ix.seq_of_query[q] : q;
        const int blk = pos / ix.page;
        if (blk >= ix.max_blocks) return -1;
        const int pg = ix.block_table[(size_t)seq * ix.max_blocks + blk];
        if (pg < 0) return -1;
        pos = pg * ix.page + (pos - blk * ix.page);
    }
    if (ix.N > 0 && pos >= ix.N) return -1;
    return pos;
}
