// The cache: sequence slots, pages of key/value storage for groups of layers, fixed-size state per sequence.
//
// The reference keeps ONE sequence whose key/value tensors are re-allocated and copied on every decoded token
// (examples/common/llama/llama_engine.h:45-57, llama_engine.cpp:442-446).  Here a batch of sequences each owns a slot; a
// slot owns pages of VM_PAGE_TOKENS tokens out of a fixed pool, so the memory is sized by the number of tokens alive, not
// by slots x longest context.  A mixer declares what it needs to remember per sequence as a CacheNeed; layers with equal
// needs share a group (one pool of pages, one block table per slot); groups with different needs (all keys / a window)
// have storage and bookkeeping of their own.
//
// Both allocators refuse misuse loudly (a page or slot freed twice, or one that was never handed out).
#include <algorithm>
#include <set>

#include "velomind_b200/kernels.h"
#include "velomind_b200/velomind.h"

namespace vmb {

// ------------------------------------------------------------------------------------------------ FreeList
FreeList::FreeList(int n, std::string what) : n_(n), what_(std::move(what)), held_(static_cast<size_t>(std::max(n, 0)), 0) {
    free_.reserve(static_cast<size_t>(std::max(n, 0)));
    for (int i = n - 1; i >= 0; --i) free_.push_back(i);
}

int FreeList::take() {
    if (free_.empty()) throw CacheError(format("out of %ss: all %d are in use", what_.c_str(), n_));
    const int i = free_.back();
    free_.pop_back();
    if (held_[i]) throw CacheError(format("%s %d was on the free list while held", what_.c_str(), i));
    held_[i] = 1;
    return i;
}

std::vector<int> FreeList::take_many(int k) {
    if (k > static_cast<int>(free_.size()))
        throw CacheError(format("out of %ss: %d wanted, %zu of %d free", what_.c_str(), k, free_.size(), n_));
    std::vector<int> out;
    for (int j = 0; j < k; ++j) out.push_back(take());
    return out;
}

void FreeList::give(int i) {
    if (i < 0 || i >= n_) throw CacheError(format("%s %d does not exist (0..%d)", what_.c_str(), i, n_ - 1));
    if (!held_[i]) throw CacheError(format("%s %d is given back but was not held (freed twice?)", what_.c_str(), i));
    held_[i] = 0;
    // keep "lowest first": the list is sorted descending, back() is the lowest free id
    auto pos = std::lower_bound(free_.begin(), free_.end(), i, std::greater<int>());
    free_.insert(pos, i);
}

void FreeList::check() const {
    std::vector<int> seen(static_cast<size_t>(n_), 0);
    for (int i : free_) {
        if (i < 0 || i >= n_) throw CacheError(format("%s %d on the free list does not exist", what_.c_str(), i));
        ++seen[i];
    }
    for (int i = 0; i < n_; ++i)
        if (seen[i] + (held_[i] ? 1 : 0) != 1)
            throw CacheError(format("%s %d: on the free list %d times, held=%d", what_.c_str(), i, seen[i], static_cast<int>(held_[i])));
}

// ------------------------------------------------------------------------------------------------ PageBook
static int ceil_div(int a, int b) { return (a + b - 1) / b; }

PageBook::PageBook(const CacheNeed& need_, int n_pages_, int max_slots_, int max_blocks_)
    : need(need_), n_pages(n_pages_), max_slots(max_slots_), max_blocks(max_blocks_), pages(n_pages_, "cache page"),
      blocks_begin(static_cast<size_t>(max_slots_), 0), blocks_end(static_cast<size_t>(max_slots_), 0),
      table_(static_cast<size_t>(max_slots_) * max_blocks_, -1) {
    if (need.kind != CacheNeed::All && need.kind != CacheNeed::Window) throw CacheError("a cache group holds keys and values; a need of kind 'none' has none");
    if (need.kind == CacheNeed::Window && need.window <= 0) throw CacheError("a window group needs window > 0");
    if (need.key_dim != need.value_dim)
        throw CacheError(format("a cache group stores keys and values of one head size; a mixer asked for keys of %d and values of %d", need.key_dim,
                                need.value_dim));
}

int PageBook::pages_needed(int slot, int new_len) const { return std::max(0, ceil_div(new_len, VM_PAGE_TOKENS) - blocks_end[slot]); }

void PageBook::ensure(int slot, int new_len) {
    const int want = ceil_div(new_len, VM_PAGE_TOKENS);
    if (want > max_blocks) throw CacheError(format("a sequence of %d tokens needs %d blocks; the table holds %d", new_len, want, max_blocks));
    const int k = want - blocks_end[slot];
    if (k <= 0) return;
    const std::vector<int> ids = pages.take_many(k);
    for (int j = 0; j < k; ++j) table_[static_cast<size_t>(slot) * max_blocks + blocks_end[slot] + j] = ids[j];
    blocks_end[slot] = want;
    ++version;
}

void PageBook::trim(int slot, int length) {
    if (need.kind != CacheNeed::Window) return;
    // the next query sits at position `length` or later and sees keys at positions > length - window
    const int first_needed = std::max(0, length - need.window + 1);
    int b = blocks_begin[slot];
    while (b < blocks_end[slot] && (b + 1) * VM_PAGE_TOKENS <= first_needed) {
        int& entry = table_[static_cast<size_t>(slot) * max_blocks + b];
        pages.give(entry);
        entry = -1;
        ++b;
        ++version;
    }
    blocks_begin[slot] = b;
}

void PageBook::release(int slot) {
    for (int b = blocks_begin[slot]; b < blocks_end[slot]; ++b) {
        int& entry = table_[static_cast<size_t>(slot) * max_blocks + b];
        pages.give(entry);
        entry = -1;
    }
    blocks_begin[slot] = 0;
    blocks_end[slot] = 0;
    ++version;
}

// ------------------------------------------------------------------------------------------------ CacheBook
static int slots_for(long long max_tokens, int max_slots) {
    if (max_tokens < VM_PAGE_TOKENS) throw CacheError(format("max_tokens %lld is less than one page of %d tokens", max_tokens, VM_PAGE_TOKENS));
    const long long pages = max_tokens / VM_PAGE_TOKENS;
    return max_slots > 0 ? max_slots : static_cast<int>(std::min<long long>(pages, 4096));
}

CacheBook::CacheBook(const std::vector<CacheNeed>& needs, const std::vector<int>& shares, long long max_tokens, int max_positions_, int max_slots_)
    : n_pages(static_cast<int>(std::max<long long>(max_tokens, 0) / VM_PAGE_TOKENS)), max_positions(max_positions_),
      max_blocks(ceil_div(max_positions_, VM_PAGE_TOKENS)), max_slots(slots_for(max_tokens, max_slots_)), slots(max_slots, "sequence slot"),
      length(static_cast<size_t>(max_slots), 0) {
    const size_t n = needs.size();
    std::vector<std::pair<int, int>> of_run(n, {-1, -1});
    for (size_t i = 0; i < n; ++i) {
        const CacheNeed& need = needs[i];
        if (shares[i] >= 0 || need.kind == CacheNeed::None) continue;
        int g = -1;
        for (size_t j = 0; j < groups.size(); ++j)
            if (groups[j].need.same_group(need)) g = static_cast<int>(j);
        if (g < 0) {
            groups.emplace_back(need, n_pages, max_slots, max_blocks);
            layers_in_group.push_back(0);
            g = static_cast<int>(groups.size()) - 1;
        }
        of_run[i] = {g, layers_in_group[g]++};
    }
    where_.resize(n);
    state_floats.assign(n, 0);
    state_owner.assign(n, -1);
    for (size_t i = 0; i < n; ++i) {
        const int owner = shares[i] >= 0 ? shares[i] : static_cast<int>(i);
        where_[i] = of_run[owner];
        if (needs[owner].state_floats > 0) {
            state_floats[i] = needs[owner].state_floats;
            state_owner[i] = owner;
        }
    }
}

int CacheBook::open() {
    const int slot = slots.take();
    length[slot] = 0;
    return slot;
}

void CacheBook::close(int slot) {
    if (!slots.is_held(slot)) throw CacheError(format("sequence slot %d is closed but was not open", slot));
    for (auto& g : groups) g.release(slot);
    length[slot] = 0;
    slots.give(slot);
}

bool CacheBook::can_hold(const std::vector<std::pair<int, int>>& slot_new_len) const {
    for (const auto& g : groups) {
        long long need = 0;
        for (const auto& sn : slot_new_len) need += g.pages_needed(sn.first, sn.second);
        if (need > g.pages.free_count()) return false;
    }
    return true;
}

void CacheBook::reserve(int slot, int new_len) {
    if (!slots.is_held(slot)) throw CacheError(format("sequence slot %d is not open", slot));
    if (new_len > max_positions) throw CacheError(format("sequence would reach %d tokens; the model's limit is %d", new_len, max_positions));
    for (const auto& g : groups)
        if (g.pages_needed(slot, new_len) > g.pages.free_count())
            throw CacheError(format("out of cache pages: slot %d needs %d more pages of %d tokens, %d of %d free", slot, g.pages_needed(slot, new_len),
                                    VM_PAGE_TOKENS, g.pages.free_count(), g.n_pages));
    for (auto& g : groups) g.ensure(slot, new_len);
}

void CacheBook::commit(int slot, int new_len) {
    length[slot] = new_len;
    for (auto& g : groups) g.trim(slot, new_len);
}

long long CacheBook::tokens_held() const {
    int most = 0;
    for (const auto& g : groups) most = std::max(most, g.pages.held_count());
    return static_cast<long long>(most) * VM_PAGE_TOKENS;
}

void CacheBook::check() const {
    slots.check();
    for (const auto& g : groups) {
        g.pages.check();
        std::set<int> held;
        for (int s = 0; s < max_slots; ++s)
            for (int b = 0; b < g.max_blocks; ++b) {
                const int pg = g.table_row(s)[b];
                const bool inside = g.blocks_begin[s] <= b && b < g.blocks_end[s];
                if ((pg >= 0) != inside)
                    throw CacheError(format("slot %d block %d: page %d but live range is [%d, %d)", s, b, pg, g.blocks_begin[s], g.blocks_end[s]));
                if (pg >= 0) {
                    if (!held.insert(pg).second) throw CacheError(format("cache page %d is held twice", pg));
                    if (!slots.is_held(s)) throw CacheError(format("cache page %d belongs to closed slot %d", pg, s));
                }
            }
        if (static_cast<int>(held.size()) != g.pages.held_count())
            throw CacheError(format("%d pages are marked held but block tables name %zu", g.pages.held_count(), held.size()));
    }
}

// ------------------------------------------------------------------------------------------------ SequenceCache
SequenceCache::SequenceCache(const std::vector<CacheNeed>& needs, const std::vector<int>& shares, long long max_tokens, int max_positions,
                             DType dtype_, cudaStream_t stream, int max_slots)
    : book(needs, shares, max_tokens, max_positions, max_slots), dtype(dtype_), stream_(stream) {
    for (size_t g = 0; g < book.groups.size(); ++g) {
        const CacheNeed& need = book.groups[g].need;
        GroupStorage s;
        s.layer_bytes = static_cast<size_t>(book.n_pages) * need.kv_heads * VM_PAGE_TOKENS * need.key_dim * dtype_size(dtype);
        s.k = std::make_unique<DeviceBuffer>(s.layer_bytes * book.layers_in_group[g], /*zero=*/true);
        s.v = std::make_unique<DeviceBuffer>(s.layer_bytes * book.layers_in_group[g], /*zero=*/true);
        storage.push_back(std::move(s));
    }
    state.resize(needs.size());
    for (size_t i = 0; i < needs.size(); ++i) {
        const int owner = book.state_owner[i];
        if (owner < 0) continue;
        if (owner == static_cast<int>(i))
            state[i] = std::make_shared<DeviceBuffer>(static_cast<size_t>(book.max_slots) * book.state_floats[i] * sizeof(float), /*zero=*/true);
        else state[i] = state[owner];
    }
}

int SequenceCache::open() {
    const int slot = book.open();
    for (size_t i = 0; i < state.size(); ++i)
        if (state[i] && book.state_owner[i] == static_cast<int>(i)) {
            const size_t row = static_cast<size_t>(book.state_floats[i]) * sizeof(float);
            if (cudaMemsetAsync(static_cast<char*>(state[i]->ptr) + row * slot, 0, row, stream_) != cudaSuccess) {
                book.close(slot);
                throw KernelError("could not clear a sequence's state area");
            }
        }
    return slot;
}

void* SequenceCache::k_pages(int group, int layer) const { return static_cast<char*>(storage[group].k->ptr) + storage[group].layer_bytes * layer; }
void* SequenceCache::v_pages(int group, int layer) const { return static_cast<char*>(storage[group].v->ptr) + storage[group].layer_bytes * layer; }

}  // namespace vmb
