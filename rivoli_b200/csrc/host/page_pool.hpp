// Host-side KV page allocator: a LIFO free list of fixed-size pages plus one block table
// per sequence. The reference keeps contiguous per-layer slabs sized max_ctx
// (crates/engine/src/glm/engine.rs:77-83,167-175) and has no pager; the free-list idiom
// follows its expert arena (crates/core/src/arena.rs:131-149): alloc pops the tail, free
// pushes, so the mapping is a pure function of the call history and page tables are
// reproducible bit for bit.
#pragma once

#include <cstdint>
#include <vector>

namespace rivoli {

class PagePool {
public:
    PagePool(int n_pages, int n_seqs, int max_pages_per_seq, int page_tokens);

    // Seeded Fisher-Yates over the current free list (splitmix64; j = r % (i + 1), i descending).
    void shuffle(uint64_t seed);
    // Grow `seq` to hold n_tokens. 0 ok; 1001 bad seq; 1002 block-table row full;
    // 1007 pool exhausted (nothing mapped in that case).
    int reserve(int seq, int n_tokens);
    // Return every page of `seq` to the free list, logical page 0 first.
    int release(int seq);

    int n_free() const { return (int)free_.size(); }
    int n_pages() const { return n_pages_; }
    int n_seqs() const { return n_seqs_; }
    int max_pages_per_seq() const { return max_pages_; }
    int page_tokens() const { return page_tokens_; }
    int seq_pages(int seq) const { return seq_pages_[seq]; }
    const int32_t* block_table() const { return table_.data(); }
    const int32_t* free_list() const { return free_.data(); }

private:
    int n_pages_, n_seqs_, max_pages_, page_tokens_;
    std::vector<int32_t> free_;
    std::vector<int32_t> table_;
    std::vector<int32_t> seq_pages_;
};

}  // namespace rivoli
