// The cache manager: keys and values in pages, a block table per request and
// group, and slots for per-request state of fixed size.
//
// What it owns.  Cache *units* (one per entry of the run order that writes keys
// and values) are sorted into *groups* by what they need: number of key/value
// heads, head size and attention window.  Each group has pages of its own (one
// device array [unit, page, K|V, kv_head, slot, head_dim] and one free list) and
// one block table per request, shared by the group's units, so a page id means the
// same positions in every unit of the group.  Pages return to the free list when a
// request closes, when it is cut back, and, in a windowed group, as soon as no
// later query can see them; freed pages are handed out again, most recently freed
// first.
//
// The reference keeps one `KvCache` per sequence with groups by window, a page
// table per group, on-demand mapping in `reserve()`, `truncate()`, windowed
// release and `clear()` (include/liyab/kv_cache.h:10-32, 72-428;
// src/core/kv_cache.cpp:186-265, 418-439, 474-515) and keeps recurrent state
// beside the cache in the sequence's context (src/core/transformer.h:854-865,
// 1283-1308).  Here one pool serves all requests, which is what lets a finished
// request's pages serve the next one.
//
// Bookkeeping is host-side and runs without a GPU; only the storage lives on the
// device (and only when asked for).  Every open request has a *row* (its state
// slot); tables and lengths are arrays indexed by row.
//
// Invariant of a request's table in a group: logical pages below `released` are
// unmapped for good, pages in [released, n_logical) are all mapped, and nothing
// exists beyond n_logical.
#pragma once

#include <cstdint>
#include <map>
#include <optional>
#include <unordered_map>
#include <vector>

#include "device.h"
#include "status.h"

namespace liyab {

constexpr int32_t kUnmapped = -1;
using RequestId = int64_t;

// What one cache unit stores per position.
struct KvNeed {
    int n_kv_head = 0;
    int head_dim = 0;
    int window = 0;          // 0: every position is kept; w: the w latest positions
    auto operator<=>(const KvNeed&) const = default;
};

// Per-request state of fixed size for one unit (e.g. a recurrent mixer).
struct StateNeed {
    std::vector<int64_t> shape;
    DType dtype = DType::F32;
    size_t bytes() const;
};

// Free list over ids 0 .. n-1 with its invariants checked on every move.
class PagePool {
public:
    explicit PagePool(int num_pages);
    int num_pages() const { return num_pages_; }
    int free_count() const { return static_cast<int>(free_.size()); }
    int held_count() const { return num_pages_ - free_count(); }
    int take();                    // OutOfPages when empty
    void give_back(int page);      // INTERNAL when the page is not held
    void check() const;            // no page lost, none held twice, none free twice

private:
    int num_pages_;
    std::vector<int> free_;        // back() is handed out next
    std::vector<char> held_;
};

// Units with the same needs: one storage array, one free list, one table row per request.
class KvGroup {
public:
    KvGroup(KvNeed need, std::vector<int> units, int page_size, int num_pages, int max_requests);

    KvNeed need;
    std::vector<int> units;
    int page_size;
    PagePool pool;
    std::vector<std::vector<int32_t>> table;     // [row][logical page]
    std::vector<int64_t> n_logical;              // pages a row's table spans
    std::vector<int64_t> released;               // pages below this were freed by the window
    DeviceBuffer storage;
    DType storage_dtype = DType::F32;

    int unit_index(int unit) const;
    size_t unit_bytes() const;                   // bytes of one unit's pages
    void* unit_storage(int unit) const;
    size_t bytes_per_token(size_t element_size) const;
    int64_t pages_for(int64_t end) const { return (end + page_size - 1) / page_size; }
    int64_t pages_needed(int row, int64_t end) const;
    void map_row(int row, int64_t end);
    void release_unreachable(int row, int64_t length);
    void truncate_row(int row, int64_t length, RequestId request);
    void clear_row(int row);
};

// Slots of fixed size, one per live request, for units that keep state.  A request's slot is
// also its row in the cache manager's tables.
class StateSlots {
public:
    StateSlots(std::map<int, StateNeed> needs, int n_slots);
    std::map<int, StateNeed> needs;
    int n_slots;
    PagePool pool;
    std::unordered_map<RequestId, int> slot_of;
    std::map<int, DeviceBuffer> storage;         // unit -> [slot, ...]

    void allocate_storage();
    int open(RequestId request, cudaStream_t stream);
    void close(RequestId request);
};

class CacheManager {
public:
    // `with_storage`: allocate the pages and state slots on the current device.
    // `pages_per_group` overrides num_pages for groups with that need.
    CacheManager(const std::map<int, KvNeed>& kv_needs, const std::map<int, StateNeed>& state_needs, int page_size,
                 int num_pages, int max_requests, DType dtype, bool with_storage,
                 const std::map<KvNeed, int>& pages_per_group = {});

    int page_size;
    int max_requests;
    DType dtype;
    StateSlots states;
    std::vector<int64_t> length_of_row;
    std::vector<KvGroup> groups;
    std::map<int, int> group_of_unit;
    bool windowed = false;
    cudaStream_t stream = nullptr;               // where state slots are cleared at open

    // -- requests
    void open(RequestId request);
    void close(RequestId request);
    bool is_open(RequestId request) const { return states.slot_of.count(request) != 0; }
    int row_of(RequestId request) const;         // INVALID_ARGUMENT when not open
    int64_t length(RequestId request) const { return length_of_row[static_cast<size_t>(row_of(request))]; }
    size_t open_count() const { return states.slot_of.size(); }

    // -- reserving and committing, by row
    // Per group, the pages that appending n_new[i] tokens to rows[i] would take, summed over the rows.
    std::vector<int64_t> need_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new) const;
    bool can_reserve_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new) const;
    // Maps pages for positions [length, length + n_new) of every row in every group, or none at all.
    void reserve_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new);
    // The step ran: the rows are n_new tokens longer; windows move on.
    void commit_rows(const std::vector<int>& rows, const std::vector<int64_t>& n_new);
    // Undoes reserve_rows after a failed step: pages beyond each row's length go back.
    void rollback_rows(const std::vector<int>& rows);

    // -- the same by request
    void reserve(RequestId request, int64_t n_new);
    void commit(RequestId request, int64_t n_new);
    void truncate(RequestId request, int64_t length);

    // -- what a step needs
    // The block tables of `rows`, row-major [rows.size(), width] (width 0: the widest of them).
    std::vector<int32_t> table_rows(int group, const std::vector<int>& rows, int* width) const;
    int32_t slot_of(int group, int row, int64_t position) const;

    // -- accounting
    std::vector<int> pages_in_use() const;
    std::vector<int> free_pages() const;
    size_t bytes_per_token() const;
    // Every held page is in exactly one table, pools are consistent, rows of closed requests are empty.
    void check() const;
};

}  // namespace liyab
