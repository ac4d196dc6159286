// page_pool.hpp — host-side page bookkeeping of the shared KV pool.
//
// Observable state (block tables, reference counts, the ORDER of the free-page
// stack and of the free-slice stack, cow_count, the one-shot copy request) is
// kept identical, operation by operation, to nova::KvPool of the reference
// (code/graph/kv_pool.h:68-197).  The rules that matter for that:
//   * init(): pages are stacked NB-1 … 0 and handed out from the top, so page 0
//     goes first; slices likewise (kv_pool.h:70-84).
//   * acquire(): slice `id` pre-reserves its identity pages id*nblocks+b, each
//     set to refcount 1 and taken out of the free stack wherever it sits,
//     keeping the order of the rest (kv_pool.h:90-113).
//   * free_page(): a count that reaches zero (or below) is clamped to zero and
//     the page pushed on top of the stack — LIFO reuse (kv_pool.h:123-126).
//   * attach_prefix(): overwrites the first ceil(n/kb) entries of dst with src's
//     and bumps their counts; dst's own identity pages for those entries stay
//     reserved and unreachable (kv_pool.h:141-148).
//   * cow(): a shared page (count > 1) is replaced by a freshly allocated one;
//     the request (from, to) is left for the device copy (kv_pool.h:153-166).
//   * release(): every table entry is un-referenced, the slice id is pushed on
//     the slice stack (kv_pool.h:168-174).
// Slices are addressed by id, not by pointer, so the reference's pointer
// invalidation on release (docs/API.md:327-329) has no counterpart here.
#pragma once
#include <cstdint>
#include <vector>

namespace novab {

struct SliceState {
    int id = -1;
    int copy_from = -1;      // KvSlice::need_copy_from
    int copy_to = -1;        // KvSlice::need_copy_blk
    int64_t n_past = 0;
    std::vector<int32_t> table;   // logical block -> physical page
};

class PagePool {
public:
    explicit PagePool(int kv_block = 16) { set_block(kv_block); }

    bool set_block(int kv_block) {
        int sh = 0;
        while ((1 << sh) < kv_block) ++sh;
        if ((1 << sh) != kv_block || kv_block < 8 || kv_block > 64) return false;
        kb_ = kv_block;
        shift_ = sh;
        return true;
    }
    int kv_block() const { return kb_; }
    int block_index(int64_t pos) const { return (int)(pos >> shift_); }   // kv_block_index
    int slot_index(int64_t pos) const { return (int)(pos & (kb_ - 1)); }  // kv_slot_index

    void init(int n_slices, int64_t ctx) {
        ctx_ = ctx;
        nblocks_ = (int)((ctx + kb_ - 1) / kb_);
        live_.clear();
        slice_stack_.clear();
        for (int s = n_slices; s-- > 0;) slice_stack_.push_back(s);
        nb_total_ = n_slices * nblocks_;
        refs_.assign((size_t)nb_total_, 0);
        page_stack_.resize((size_t)nb_total_);
        for (int i = 0; i < nb_total_; ++i) page_stack_[(size_t)i] = nb_total_ - 1 - i;
        cow_count_ = 0;
    }

    // Returns the slice id, or -1 when every slice is taken.
    int acquire() {
        if (slice_stack_.empty()) return -1;
        const int id = slice_stack_.back();
        slice_stack_.pop_back();
        SliceState st;
        st.id = id;
        st.table.resize((size_t)nblocks_);
        const int first = id * nblocks_;
        for (int b = 0; b < nblocks_; ++b) st.table[(size_t)b] = first + b;
        // Reserve the identity pages.  The reference erases, for each page in turn,
        // the FIRST entry of the stack that names it (std::find + erase).  A page
        // can sit in the stack twice after a double un-reference, and then the
        // second entry survives.  One pass that drops the first entry seen of
        // each identity page leaves exactly the same stack.
        const int last = first + nblocks_;
        std::vector<char> dropped((size_t)nblocks_, 0);
        size_t w = 0;
        for (size_t r = 0; r < page_stack_.size(); ++r) {
            const int pg = page_stack_[r];
            if (pg >= first && pg < last && !dropped[(size_t)(pg - first)]) {
                dropped[(size_t)(pg - first)] = 1;
                continue;
            }
            page_stack_[w++] = pg;
        }
        page_stack_.resize(w);
        for (int pg = first; pg < last && pg < nb_total_; ++pg) refs_[(size_t)pg] = 1;
        live_.push_back(std::move(st));
        return id;
    }

    int alloc_page() {
        if (page_stack_.empty()) return -1;
        const int pg = page_stack_.back();
        page_stack_.pop_back();
        refs_[(size_t)pg] = 1;
        return pg;
    }
    void free_page(int pg) {
        if (pg < 0 || pg >= nb_total_) return;
        int& r = refs_[(size_t)pg];
        r -= 1;
        if (r <= 0) {
            r = 0;
            page_stack_.push_back(pg);
        }
    }
    void ref_page(int pg) {
        if (pg >= 0 && pg < nb_total_) refs_[(size_t)pg] += 1;
    }
    int refcnt(int pg) const { return (pg >= 0 && pg < nb_total_) ? refs_[(size_t)pg] : 0; }

    // Share the first k logical blocks of src with dst.
    bool attach(int dst, int src, int k) {
        SliceState* d = find(dst);
        const SliceState* s = find(src);
        if (!d || !s || k < 0 || k > nblocks_) return false;
        for (int i = 0; i < k; ++i) {
            d->table[(size_t)i] = s->table[(size_t)i];
            ref_page(s->table[(size_t)i]);
        }
        if (k > 0) d->n_past = (int64_t)k * kb_;   // set inside the reference's loop: untouched when k == 0
        return true;
    }

    // Share the first n_tokens positions (a partly filled tail page included).
    bool attach_prefix(int dst, int src, int64_t n_tokens) {
        SliceState* d = find(dst);
        const SliceState* s = find(src);
        if (!d || !s || n_tokens < 0) return false;
        int64_t nb = (n_tokens + kb_ - 1) / kb_;
        if (nb > nblocks_) nb = nblocks_;
        for (int64_t i = 0; i < nb; ++i) {
            d->table[(size_t)i] = s->table[(size_t)i];
            ref_page(s->table[(size_t)i]);
        }
        d->n_past = n_tokens;
        return true;
    }

    // -1: nothing to copy; -2: pool exhausted; otherwise the new private page.
    int cow(int slice, int64_t pos) {
        SliceState* st = find(slice);
        if (!st) return -1;
        const int lb = block_index(pos);
        if (pos < 0 || lb >= (int)st->table.size()) return -1;
        const int shared = st->table[(size_t)lb];
        if (refcnt(shared) <= 1) return -1;
        const int fresh = alloc_page();
        if (fresh < 0) return -2;
        cow_count_ += 1;
        st->copy_from = shared;
        st->copy_to = fresh;
        st->table[(size_t)lb] = fresh;
        free_page(shared);
        return fresh;
    }

    bool release(int slice) {
        for (size_t i = 0; i < live_.size(); ++i) {
            if (live_[i].id != slice) continue;
            for (int32_t pg : live_[i].table) free_page(pg);
            slice_stack_.push_back(slice);
            live_.erase(live_.begin() + (std::ptrdiff_t)i);
            return true;
        }
        return false;
    }

    SliceState* find(int slice) {
        for (auto& s : live_) if (s.id == slice) return &s;
        return nullptr;
    }
    const SliceState* find(int slice) const {
        for (const auto& s : live_) if (s.id == slice) return &s;
        return nullptr;
    }

    // The slice id the next acquire() hands out (-1: none left).  Does not change anything.
    int next_slice() const { return slice_stack_.empty() ? -1 : slice_stack_.back(); }

    // Entries of OTHER live tables that map one of `slice`'s identity pages (slice*nblocks + b): pages a
    // fork still reads after its parent was released, or pages handed out by cow() while the slice was free.
    // acquire() sets the count of every identity page to 1 whatever it was (kv_pool.h:100-112), so acquiring a
    // slice for which this is non-zero would let two sessions write the same pages; callers check first.
    int foreign_mappings(int slice) const {
        const int first = slice * nblocks_, last = first + nblocks_;
        int n = 0;
        for (const auto& s : live_) {
            if (s.id == slice) continue;
            for (int32_t pg : s.table) n += (pg >= first && pg < last) ? 1 : 0;
        }
        return n;
    }

    int nblocks() const { return nblocks_; }
    int nb_total() const { return nb_total_; }
    int64_t ctx() const { return ctx_; }
    int cow_count() const { return cow_count_; }
    int free_pages() const { return (int)page_stack_.size(); }
    int free_slices() const { return (int)slice_stack_.size(); }
    int used() const { return (int)live_.size(); }
    const std::vector<int>& refs() const { return refs_; }
    const std::vector<int>& page_stack() const { return page_stack_; }
    const std::vector<int>& slice_stack() const { return slice_stack_; }
    const std::vector<SliceState>& live() const { return live_; }

private:
    int kb_ = 16, shift_ = 4;
    int64_t ctx_ = 0;
    int nblocks_ = 0, nb_total_ = 0, cow_count_ = 0;
    std::vector<SliceState> live_;      // in acquisition order
    std::vector<int> slice_stack_;      // back = next slice id
    std::vector<int> page_stack_;       // back = next page
    std::vector<int> refs_;
};

}  // namespace novab
