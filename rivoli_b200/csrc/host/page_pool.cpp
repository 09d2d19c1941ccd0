#include "page_pool.hpp"

#include "../../../include/rivoli_kernels.h"

namespace rivoli {

static uint64_t splitmix64(uint64_t& s) {
    uint64_t z = (s += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

PagePool::PagePool(int n_pages, int n_seqs, int max_pages_per_seq, int page_tokens)
    : n_pages_(n_pages), n_seqs_(n_seqs), max_pages_(max_pages_per_seq), page_tokens_(page_tokens),
      free_((size_t)n_pages), table_((size_t)n_seqs * max_pages_per_seq, -1), seq_pages_((size_t)n_seqs, 0) {
    for (int i = 0; i < n_pages; ++i) free_[(size_t)i] = n_pages - 1 - i;  // first pops: 0, 1, 2, ...
}

void PagePool::shuffle(uint64_t seed) {
    uint64_t s = seed;
    for (int i = (int)free_.size() - 1; i > 0; --i) {
        const int j = (int)(splitmix64(s) % (uint64_t)(i + 1));
        std::swap(free_[(size_t)i], free_[(size_t)j]);
    }
}

int PagePool::reserve(int seq, int n_tokens) {
    if (seq < 0 || seq >= n_seqs_ || n_tokens < 0) return 1001;
    const int need = (n_tokens + page_tokens_ - 1) / page_tokens_;
    if (need > max_pages_) return 1002;
    const int have = seq_pages_[(size_t)seq];
    if (need - have > (int)free_.size()) return 1007;
    for (int i = have; i < need; ++i) {
        table_[(size_t)seq * max_pages_ + i] = free_.back();
        free_.pop_back();
    }
    if (need > have) seq_pages_[(size_t)seq] = need;
    return 0;
}

int PagePool::release(int seq) {
    if (seq < 0 || seq >= n_seqs_) return 1001;
    for (int i = 0; i < seq_pages_[(size_t)seq]; ++i) {
        int32_t& e = table_[(size_t)seq * max_pages_ + i];
        free_.push_back(e);
        e = -1;
    }
    seq_pages_[(size_t)seq] = 0;
    return 0;
}

}  // namespace rivoli

// ---- C ABI ------------------------------------------------------------------------------------
#define RV_HOST_API extern "C" __attribute__((visibility("default")))
using rivoli::PagePool;

RV_HOST_API void* rivoli_pagepool_create(int n_pages, int n_seqs, int max_pages_per_seq, int page_tokens) {
    if (n_pages <= 0 || n_seqs <= 0 || max_pages_per_seq <= 0 || page_tokens <= 0) return nullptr;
    return new PagePool(n_pages, n_seqs, max_pages_per_seq, page_tokens);
}
RV_HOST_API void rivoli_pagepool_destroy(void* p) { delete static_cast<PagePool*>(p); }
RV_HOST_API void rivoli_pagepool_shuffle(void* p, uint64_t seed) { static_cast<PagePool*>(p)->shuffle(seed); }
RV_HOST_API int rivoli_pagepool_reserve(void* p, int seq, int n_tokens) {
    return p ? static_cast<PagePool*>(p)->reserve(seq, n_tokens) : 1001;
}
RV_HOST_API int rivoli_pagepool_release(void* p, int seq) {
    return p ? static_cast<PagePool*>(p)->release(seq) : 1001;
}
RV_HOST_API int rivoli_pagepool_n_free(const void* p) { return static_cast<const PagePool*>(p)->n_free(); }
RV_HOST_API int rivoli_pagepool_seq_pages(const void* p, int seq) {
    return static_cast<const PagePool*>(p)->seq_pages(seq);
}
RV_HOST_API const int32_t* rivoli_pagepool_block_table(const void* p) {
    return static_cast<const PagePool*>(p)->block_table();
}
RV_HOST_API const int32_t* rivoli_pagepool_free_list(const void* p) {
    return static_cast<const PagePool*>(p)->free_list();
}
