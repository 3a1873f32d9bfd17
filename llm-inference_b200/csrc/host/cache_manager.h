// Host-side bookkeeping of the paged key/value cache and of per-request state slots.
//
// Layers that share a key/value shape and a window form a group; each group has its own
// pool of physical pages and each request has, per group, a block table from logical page
// (position / page_size) to physical page. A request is admitted only when every group can
// promise the pages its whole budget needs, so a request that starts can always finish
// (python/instinct/mlx_engine.py:262-306; src/kv_cache.cpp:38-73). Pages are materialised
// as positions are reached, given back when the request ends, and - in a windowed group -
// as soon as no later position can see them (mlx_engine.py:349-372); freed pages go back to
// the pool and are handed out again, lowest id first (python/instinct/paged_kv.py:79-153).
// Beside pages, a request may hold one slot of fixed-size state (paged_kv.py:296-313).
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace b200 {

using RequestId = std::int64_t;

struct CacheError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class PagePool {
 public:
  explicit PagePool(int capacity);

  int capacity() const { return capacity_; }
  int free_pages() const { return static_cast<int>(free_.size()); }
  int available() const { return free_pages() - reserved_; }
  int used() const { return capacity_ - free_pages(); }
  int reserved() const { return reserved_; }
  int high_water() const { return high_water_; }
  int refcount(int page) const { return refs_.at(page); }

  bool reserve(int count);
  void unreserve(int count);
  // Takes the lowest free page, from the caller's reservation if `from_reservation`.
  int allocate(bool from_reservation);
  void retain(int page);
  void release(int page);

 private:
  int capacity_;
  int reserved_{0};
  int high_water_{0};
  std::vector<int> free_;  // min-heap
  std::vector<int> refs_;
};

struct GroupSpec {
  std::string name;
  int capacity_pages{0};
  int window{0};  // 0: every earlier position stays visible
};

struct GroupStats {
  std::string name;
  int window{0};
  int capacity_pages{0};
  int used_pages{0};
  int reserved_pages{0};
  int free_pages{0};
  int high_water{0};
};

struct CacheStats {
  std::vector<GroupStats> groups;
  std::int64_t live_tokens{0};
  std::int64_t internal_fragmentation_tokens{0};
  std::int64_t allocation_failures{0};
  int state_slots{0};
  int free_state_slots{0};
  int requests{0};
};

class CacheManager {
 public:
  // `step_tokens` bounds how many positions one request can add in one step; it sizes the
  // reservation of windowed groups (window + step_tokens positions, plus one page of slack).
  CacheManager(int page_size, std::vector<GroupSpec> groups, int state_slots, int step_tokens);

  int page_size() const { return page_size_; }
  int num_groups() const { return static_cast<int>(groups_.size()); }
  const GroupSpec& group(int g) const { return groups_.at(g); }
  int group_index(const std::string& name) const;

  // Pages each group must promise a request that will hold `total_tokens` positions.
  std::vector<int> needs(int total_tokens) const;
  // Whether such a request could be admitted into an otherwise empty cache.
  bool can_ever_fit(int total_tokens) const;

  // Reserve pages (and a state slot, if the cache has any) for the request's whole budget.
  // Returns false, changing nothing, when a pool cannot promise them now.
  bool admit(RequestId id, int total_tokens);
  // Start a request with no reservation: it takes pages only as `ensure` asks for them and
  // `ensure` throws when a pool is empty. Used when the caller bounds memory itself.
  void open(RequestId id);
  bool contains(RequestId id) const { return requests_.count(id) != 0; }

  // Give the request a page for every position below `end`.
  void ensure(RequestId id, int end);
  // Positions below `length` now hold keys and values; windowed groups give back the pages
  // that no position >= length can see.
  void advance(RequestId id, int length);
  // Give back every page, the unused reservation and the slot.
  void release(RequestId id);

  const std::vector<int>& table(RequestId id, int g) const;
  int slot(RequestId id) const;
  int length(RequestId id) const;
  // Whether the slot was handed out since its last clear request (the owner of the device
  // arrays zeroes a slot when told to).
  std::vector<int> take_slots_to_clear();

  // Write request `ids[i]`'s table of group g into out[i * stride .. ], padded with `pad`.
  void fill_tables(const std::vector<RequestId>& ids, int g, std::int32_t* out, int stride,
                   std::int32_t pad) const;

  CacheStats stats() const;
  void count_allocation_failure() { ++allocation_failures_; }
  // Throws CacheError if a page is lost, held twice, or a count disagrees.
  void check_invariants() const;

 private:
  struct Entry {
    std::vector<std::vector<int>> tables;  // [group][logical page] -> physical page, -1 = given back
    std::vector<int> reserved;             // pages promised but not yet taken, per group
    std::vector<int> trimmed;              // logical pages below this index were given back
    int slot{-1};
    int length{0};
    bool has_reservation{false};
  };

  int window_pages(const GroupSpec& group) const;
  int take_page(Entry& entry, int g);
  Entry& entry(RequestId id);
  const Entry& entry(RequestId id) const;

  int page_size_;
  int step_tokens_;
  std::vector<GroupSpec> groups_;
  std::vector<PagePool> pools_;
  std::vector<int> free_slots_;
  std::vector<int> slots_to_clear_;
  int state_slots_;
  std::unordered_map<RequestId, Entry> requests_;
  std::int64_t allocation_failures_{0};
};

}  // namespace b200
