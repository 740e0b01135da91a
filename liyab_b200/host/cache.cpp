#include "cache.h"

#include <algorithm>
#include <set>

namespace liyab {

size_t StateNeed::bytes() const {
    size_t n = dtype_size(dtype);
    for (const int64_t d : shape) n *= static_cast<size_t>(d);
    return n;
}

PagePool::PagePool(int num_pages) : num_pages_(num_pages) {
    if (num_pages <= 0) throw invalid_argument("a page pool needs at least one page (got {})", num_pages);
    free_.reserve(static_cast<size_t>(num_pages));
    for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);      // page 0 is handed out first
    held_.assign(static_cast<size_t>(num_pages), 0);
}

int PagePool::take() {
    if (free_.empty()) throw OutOfPages("no free page");
    const int page = free_.back();
    free_.pop_back();
    if (held_[static_cast<size_t>(page)]) throw internal_error("page {} was on the free list while held", page);
    held_[static_cast<size_t>(page)] = 1;
    return page;
}

void PagePool::give_back(int page) {
    if (page < 0 || page >= num_pages_ || !held_[static_cast<size_t>(page)])
        throw internal_error("page {} is given back but not held", page);
    held_[static_cast<size_t>(page)] = 0;
    free_.push_back(page);
}

void PagePool::check() const {
    std::set<int> seen(free_.begin(), free_.end());
    if (seen.size() != free_.size()) throw internal_error("a page is on the free list twice");
    int held = 0;
    for (const int p : free_)
        if (held_[static_cast<size_t>(p)]) throw internal_error("page {} is both free and held", p);
    for (const char h : held_) held += h;
    if (held + static_cast<int>(free_.size()) != num_pages_) throw internal_error("a page is lost");
}

KvGroup::KvGroup(KvNeed need_, std::vector<int> units_, int page_size_, int num_pages, int max_requests)
    : need(need_), units(std::move(units_)), page_size(page_size_), pool(num_pages),
      table(static_cast<size_t>(max_requests)), n_logical(static_cast<size_t>(max_requests), 0),
      released(static_cast<size_t>(max_requests), 0) {}

int KvGroup::unit_index(int unit) const {
    const auto it = std::find(units.begin(), units.end(), unit);
    if (it == units.end()) throw internal_error("cache unit {} is not in this group", unit);
    return static_cast<int>(it - units.begin());
}

size_t KvGroup::unit_bytes() const {
    return static_cast<size_t>(pool.num_pages()) * 2 * static_cast<size_t>(need.n_kv_head) * static_cast<size_t>(page_size) *
           static_cast<size_t>(need.head_dim) * dtype_size(storage_dtype);
}

void* KvGroup::unit_storage(int unit) const {
    if (storage.data() == nullptr) throw internal_error("the cache has no device storage");
    return static_cast<char*>(storage.data()) + static_cast<size_t>(unit_index(unit)) * unit_bytes();
}

size_t KvGroup::bytes_per_token(size_t element_size) const {
    return 2 * units.size() * static_cast<size_t>(need.n_kv_head) * static_cast<size_t>(need.head_dim) * element_size;
}

int64_t KvGroup::pages_needed(int row, int64_t end) const {
    const size_t r = static_cast<size_t>(row);
    return std::max<int64_t>(pages_for(end) - std::max(n_logical[r], released[r]), 0);
}

void KvGroup::map_row(int row, int64_t end) {
    const size_t r = static_cast<size_t>(row);
    const int64_t want = pages_for(end), have = n_logical[r];
    if (want <= have) return;
    auto& t = table[r];
    t.resize(static_cast<size_t>(want), kUnmapped);
    for (int64_t j = std::max(have, released[r]); j < want; ++j)      // released pages are never mapped again
        t[static_cast<size_t>(j)] = pool.take();
    n_logical[r] = want;
}

void KvGroup::release_unreachable(int row, int64_t length) {
    // Frees the pages that no query at a position >= length can see (its earliest visible key is
    // length - window + 1).
    const int w = need.window;
    if (w <= 0) return;
    const size_t r = static_cast<size_t>(row);
    const int64_t dead = std::min(std::max<int64_t>(length - w + 1, 0) / page_size, n_logical[r]);
    for (int64_t j = released[r]; j < dead; ++j) {
        int32_t& p = table[r][static_cast<size_t>(j)];
        if (p != kUnmapped) {
            pool.give_back(p);
            p = kUnmapped;
        }
    }
    if (dead > released[r]) released[r] = dead;
}

void KvGroup::truncate_row(int row, int64_t length, RequestId request) {
    const size_t r = static_cast<size_t>(row);
    if (need.window > 0 && released[r] * page_size > std::max<int64_t>(0, length - need.window + 1))
        throw invalid_argument("request {} cannot be cut back to {}: a windowed group has already released pages that "
                               "position would need", request, length);
    const int64_t keep = pages_for(length);
    for (int64_t j = keep; j < n_logical[r]; ++j) {
        int32_t& p = table[r][static_cast<size_t>(j)];
        if (p != kUnmapped) {
            pool.give_back(p);
            p = kUnmapped;
        }
    }
    if (keep < n_logical[r]) {
        n_logical[r] = keep;
        table[r].resize(static_cast<size_t>(keep));
    }
}

void KvGroup::clear_row(int row) {
    const size_t r = static_cast<size_t>(row);
    for (const int32_t p : table[r])
        if (p != kUnmapped) pool.give_back(p);
    table[r].clear();
    n_logical[r] = 0;
    released[r] = 0;
}

StateSlots::StateSlots(std::map<int, StateNeed> needs_, int n_slots_)
    : needs(std::move(needs_)), n_slots(n_slots_), pool(n_slots_) {}

void StateSlots::allocate_storage() {
    for (const auto& [unit, need] : needs) storage[unit] = DeviceBuffer(need.bytes() * static_cast<size_t>(n_slots), true);
}

int StateSlots::open(RequestId request, cudaStream_t stream) {
    const int slot = pool.take();
    slot_of[request] = slot;
    for (auto& [unit, buf] : storage) {          // state starts at zero for every request
        const size_t n = needs.at(unit).bytes();
        if (n) LIYAB_CUDA(cudaMemsetAsync(static_cast<char*>(buf.data()) + n * static_cast<size_t>(slot), 0, n, stream));
    }
    return slot;
}

void StateSlots::close(RequestId request) {
    const auto it = slot_of.find(request);
    pool.give_back(it->second);
    slot_of.erase(it);
}

CacheManager::CacheManager(const std::map<int, KvNeed>& kv_needs, const std::map<int, StateNeed>& state_needs, int page_size_,
                           int num_pages, int max_requests_, DType dtype_, bool with_storage,
                           const std::map<KvNeed, int>& pages_per_group)
    : page_size(page_size_), max_requests(max_requests_), dtype(dtype_), states(state_needs, max_requests_),
      length_of_row(static_cast<size_t>(max_requests_), 0) {
    if (page_size <= 0) throw invalid_argument("page_size must be positive (got {})", page_size);
    std::vector<std::pair<KvNeed, std::vector<int>>> by_need;          // in order of first appearance
    for (const auto& [unit, need] : kv_needs) {
        auto it = std::find_if(by_need.begin(), by_need.end(), [&](const auto& e) { return e.first == need; });
        if (it == by_need.end()) by_need.push_back({need, {unit}});
        else it->second.push_back(unit);
    }
    for (auto& [need, units] : by_need) {
        const auto over = pages_per_group.find(need);
        const int n = over != pages_per_group.end() ? over->second : num_pages;
        for (const int u : units) group_of_unit[u] = static_cast<int>(groups.size());
        groups.emplace_back(need, units, page_size, n, max_requests);
        windowed = windowed || need.window > 0;
    }
    if (with_storage) {
        for (auto& g : groups) {
            g.storage_dtype = dtype;
            g.storage = DeviceBuffer(g.unit_bytes() * g.units.size(), true);
        }
        states.allocate_storage();
    }
}

int CacheManager::row_of(RequestId request) const {
    const auto it = states.slot_of.find(request);
    if (it == states.slot_of.end()) throw invalid_argument("request {} is not open", request);
    return it->second;
}

void CacheManager::open(RequestId request) {
    if (is_open(request)) throw make_error(Code::Busy, "request {} is already open", request);
    if (static_cast<int>(states.slot_of.size()) >= max_requests)
        throw make_error(Code::Busy, "{} requests are open already", max_requests);
    const int row = states.open(request, stream);
    length_of_row[static_cast<size_t>(row)] = 0;
}

void CacheManager::close(RequestId request) {
    const int row = row_of(request);
    for (auto& g : groups) g.clear_row(row);
    length_of_row[static_cast<size_t>(row)] = 0;
    states.close(request);
}

std::vector<int64_t> CacheManager::need_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new) const {
    std::vector<int64_t> out(groups.size(), 0);
    for (size_t g = 0; g < groups.size(); ++g)
        for (size_t i = 0; i < rows.size(); ++i)
            out[g] += groups[g].pages_needed(rows[i], length_of_row[static_cast<size_t>(rows[i])] + n_new[i]);
    return out;
}

bool CacheManager::can_reserve_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new) const {
    const auto need = need_rows(rows, n_new);
    for (size_t g = 0; g < groups.size(); ++g)
        if (need[g] > groups[g].pool.free_count()) return false;
    return true;
}

void CacheManager::reserve_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new) {
    const auto need = need_rows(rows, n_new);
    for (size_t g = 0; g < groups.size(); ++g)
        if (need[g] > groups[g].pool.free_count())
            throw OutOfPages(std::format("{} request(s) need {} more page(s) of {} positions; {} of {} are free", rows.size(),
                                         need[g], page_size, groups[g].pool.free_count(), groups[g].pool.num_pages()));
    for (auto& g : groups)
        for (size_t i = 0; i < rows.size(); ++i) g.map_row(rows[i], length_of_row[static_cast<size_t>(rows[i])] + n_new[i]);
}

void CacheManager::commit_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new) {
    for (size_t i = 0; i < rows.size(); ++i) length_of_row[static_cast<size_t>(rows[i])] += n_new[i];
    if (windowed)
        for (auto& g : groups)
            for (const int row : rows) g.release_unreachable(row, length_of_row[static_cast<size_t>(row)]);
}

void CacheManager::rollback_rows(const std::vector<int>& rows) {
    for (auto& g : groups)
        for (const int row : rows) {
            const size_t r = static_cast<size_t>(row);
            const int64_t keep = std::max(g.pages_for(length_of_row[r]), g.released[r]);
            for (int64_t j = keep; j < g.n_logical[r]; ++j) {
                int32_t& p = g.table[r][static_cast<size_t>(j)];
                if (p != kUnmapped) { g.pool.give_back(p); p = kUnmapped; }
            }
            if (keep < g.n_logical[r]) { g.n_logical[r] = keep; g.table[r].resize(static_cast<size_t>(keep)); }
        }
}

void CacheManager::reserve(RequestId request, int64_t n_new) {
    if (n_new <= 0) throw invalid_argument("request {}: a reservation needs at least one token", request);
    reserve_rows({row_of(request)}, {n_new});
}

void CacheManager::commit(RequestId request, int64_t n_new) { commit_rows({row_of(request)}, {n_new}); }

void CacheManager::truncate(RequestId request, int64_t length) {
    const int row = row_of(request);
    const int64_t have = length_of_row[static_cast<size_t>(row)];
    if (length < 0 || length > have) throw invalid_argument("request {} holds {} tokens, cannot cut to {}", request, have, length);
    if (!states.needs.empty() && length != have) throw unsupported("per-request state cannot be rolled back");
    for (auto& g : groups) g.truncate_row(row, length, request);
    length_of_row[static_cast<size_t>(row)] = length;
}

std::vector<int32_t> CacheManager::table_rows(int group, const std::vector<int>& rows, int* width) const {
    const KvGroup& g = groups.at(static_cast<size_t>(group));
    int64_t w = 1;
    for (const int row : rows) w = std::max(w, g.n_logical[static_cast<size_t>(row)]);
    if (*width > 0) {
        if (*width < w) throw invalid_argument("block table of width {} cannot hold {} pages", *width, w);
        w = *width;
    }
    *width = static_cast<int>(w);
    std::vector<int32_t> out(rows.size() * static_cast<size_t>(w), kUnmapped);
    for (size_t i = 0; i < rows.size(); ++i) {
        const auto& t = g.table[static_cast<size_t>(rows[i])];
        std::copy(t.begin(), t.end(), out.begin() + static_cast<ptrdiff_t>(i * static_cast<size_t>(w)));
    }
    return out;
}

int32_t CacheManager::slot_of(int group, int row, int64_t position) const {
    const KvGroup& g = groups[static_cast<size_t>(group)];
    const auto& t = g.table[static_cast<size_t>(row)];
    const int64_t lp = position / page_size;
    if (lp >= static_cast<int64_t>(t.size()) || t[static_cast<size_t>(lp)] < 0)
        throw internal_error("a position of the step has no page");
    return static_cast<int32_t>(static_cast<int64_t>(t[static_cast<size_t>(lp)]) * page_size + position % page_size);
}

std::vector<int> CacheManager::pages_in_use() const {
    std::vector<int> out;
    for (const auto& g : groups) out.push_back(g.pool.held_count());
    return out;
}

std::vector<int> CacheManager::free_pages() const {
    std::vector<int> out;
    for (const auto& g : groups) out.push_back(g.pool.free_count());
    return out;
}

size_t CacheManager::bytes_per_token() const {
    size_t n = 0;
    for (const auto& g : groups) n += g.bytes_per_token(dtype_size(dtype));
    return n;
}

void CacheManager::check() const {
    std::set<int> live;
    for (const auto& kv : states.slot_of) live.insert(kv.second);
    for (const auto& g : groups) {
        g.pool.check();
        std::set<int32_t> seen;
        for (int row = 0; row < max_requests; ++row) {
            const auto& t = g.table[static_cast<size_t>(row)];
            if (static_cast<int64_t>(t.size()) != g.n_logical[static_cast<size_t>(row)])
                throw internal_error("row {} has pages beyond its end", row);
            for (const int32_t p : t) {
                if (p == kUnmapped) continue;
                if (!live.count(row)) throw internal_error("row {} of a closed request still holds pages", row);
                if (!seen.insert(p).second) throw internal_error("page {} is in two tables", p);
            }
        }
        if (static_cast<int>(seen.size()) != g.pool.held_count()) throw internal_error("a held page is in no table (lost)");
    }
    states.pool.check();
}

}  // namespace liyab
