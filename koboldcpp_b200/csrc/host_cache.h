// host_cache.h -- the sequence cache shared by the decoders: which sequence owns which cache cell at which position, and which
// state slot (recurrent layers keep one fixed-size state per sequence).  Plays the part of llama_kv_cache's cell table
// (src/llama.cpp:2720-2800 llama_kv_cell / llama_kv_cache, llama_kv_cache_find_slot :3604-3740, llama_kv_cache_seq_rm :3775-3830):
// one cell table for all layers, cells found lowest-first, a closed sequence gives its cells and its slot back.  Unlike the
// reference a batch does not need one contiguous run of cells: the kernels take a cell index per token.  Host logic only.
#pragma once
#include <cstdint>
#include <vector>

namespace b200 {
namespace host {

struct SeqCache {
    struct Seq { bool open = false; bool fresh = true; int32_t len = 0; };
    std::vector<int32_t> cell_seq, cell_pos;  // per cell: owning sequence (-1: free) and position
    std::vector<Seq> seqs;                    // sequence id == state slot
    int32_t n_used = 0;                       // cells in use
    int32_t high = 0;                         // one past the highest cell in use
    int32_t first_free = 0;                   // no free cell lies below this index

    void init(int32_t n_cells, int32_t n_seq_max) {
        cell_seq.assign((size_t)n_cells, -1);
        cell_pos.assign((size_t)n_cells, -1);
        seqs.assign((size_t)n_seq_max, Seq());
        n_used = high = first_free = 0;
    }
    int32_t n_cells() const { return (int32_t)cell_seq.size(); }
    int32_t open_seq() {
        for (size_t i = 0; i < seqs.size(); i++) {
            if (!seqs[i].open) { seqs[i].open = true; seqs[i].fresh = true; seqs[i].len = 0; return (int32_t)i; }
        }
        return -1;
    }
    bool is_open(int32_t id) const { return id >= 0 && id < (int32_t)seqs.size() && seqs[(size_t)id].open; }
    void close_seq(int32_t id) {
        if (!is_open(id)) return;
        for (int32_t c = 0; c < high; c++) {
            if (cell_seq[(size_t)c] == id) {
                cell_seq[(size_t)c] = -1; cell_pos[(size_t)c] = -1; n_used--;
                if (c < first_free) first_free = c;
            }
        }
        while (high > 0 && cell_seq[(size_t)high - 1] < 0) high--;
        seqs[(size_t)id] = Seq();
    }
    // n more tokens of sequence id: their cells (lowest free first) and positions; false when the cache is full (nothing changes)
    bool place(int32_t id, int32_t n, int32_t *cells, int32_t *pos) {
        if (!is_open(id) || n < 0 || n > n_cells() - n_used) return false;
        Seq &s = seqs[(size_t)id];
        int32_t c = first_free;
        for (int32_t i = 0; i < n; i++) {
            while (cell_seq[(size_t)c] >= 0) c++;
            cell_seq[(size_t)c] = id; cell_pos[(size_t)c] = s.len;
            cells[i] = c; pos[i] = s.len++;
            if (c + 1 > high) high = c + 1;
            c++;
        }
        first_free = c;
        n_used += n;
        return true;
    }
};

}  // namespace host
}  // namespace b200
