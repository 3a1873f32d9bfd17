#include "cache_manager.h"

#include <algorithm>
#include <functional>
#include <set>

namespace b200 {

namespace {
int ceil_div(int a, int b) { return (a + b - 1) / b; }
}  // namespace

PagePool::PagePool(int capacity) : capacity_(capacity), refs_(capacity > 0 ? capacity : 0, 0) {
  if (capacity <= 0) throw CacheError("a page pool needs at least one page");
  free_.resize(capacity);
  for (int i = 0; i < capacity; ++i) free_[i] = i;
  std::make_heap(free_.begin(), free_.end(), std::greater<int>());
}

bool PagePool::reserve(int count) {
  if (count < 0) throw CacheError("cannot reserve a negative number of pages");
  if (count > available()) return false;
  reserved_ += count;
  return true;
}

void PagePool::unreserve(int count) {
  if (count < 0 || count > reserved_) throw CacheError("released more pages than were reserved");
  reserved_ -= count;
}

int PagePool::allocate(bool from_reservation) {
  if (from_reservation) {
    unreserve(1);
  } else if (available() <= 0) {
    throw CacheError("the K/V page pool is exhausted");
  }
  if (free_.empty()) throw CacheError("the K/V page pool has a reservation but no free page");
  std::pop_heap(free_.begin(), free_.end(), std::greater<int>());
  const int page = free_.back();
  free_.pop_back();
  if (refs_[page] != 0) throw CacheError("a free page still had holders");
  refs_[page] = 1;
  high_water_ = std::max(high_water_, page + 1);
  return page;
}

void PagePool::retain(int page) {
  if (page < 0 || page >= capacity_ || refs_[page] <= 0)
    throw CacheError("retained a page that isn't allocated");
  ++refs_[page];
}

void PagePool::release(int page) {
  if (page < 0 || page >= capacity_ || refs_[page] <= 0)
    throw CacheError("released a page that isn't allocated");
  if (--refs_[page] == 0) {
    free_.push_back(page);
    std::push_heap(free_.begin(), free_.end(), std::greater<int>());
  }
}

CacheManager::CacheManager(int page_size, std::vector<GroupSpec> groups, int state_slots,
                           int step_tokens)
    : page_size_(page_size), step_tokens_(step_tokens), groups_(std::move(groups)),
      state_slots_(state_slots) {
  if (page_size <= 0) throw CacheError("page size must be positive");
  if (step_tokens <= 0) throw CacheError("tokens per step must be positive");
  if (state_slots < 0) throw CacheError("state slot count cannot be negative");
  std::set<std::string> names;
  for (const auto& group : groups_) {
    if (group.window < 0) throw CacheError("a window cannot be negative");
    if (!names.insert(group.name).second) throw CacheError("duplicate cache group " + group.name);
    pools_.emplace_back(group.capacity_pages);
  }
  for (int s = state_slots - 1; s >= 0; --s) free_slots_.push_back(s);
}

int CacheManager::group_index(const std::string& name) const {
  for (int g = 0; g < num_groups(); ++g)
    if (groups_[g].name == name) return g;
  throw CacheError("unknown cache group " + name);
}

int CacheManager::window_pages(const GroupSpec& group) const {
  return ceil_div(group.window + step_tokens_, page_size_) + 1;
}

std::vector<int> CacheManager::needs(int total_tokens) const {
  std::vector<int> out;
  for (const auto& group : groups_) {
    int pages = ceil_div(total_tokens, page_size_);
    if (group.window) pages = std::min(pages, window_pages(group));
    out.push_back(pages);
  }
  return out;
}

bool CacheManager::can_ever_fit(int total_tokens) const {
  const auto need = needs(total_tokens);
  for (int g = 0; g < num_groups(); ++g)
    if (need[g] > pools_[g].capacity()) return false;
  return true;
}

bool CacheManager::admit(RequestId id, int total_tokens) {
  if (total_tokens <= 0) throw CacheError("cannot admit an empty request");
  if (contains(id)) throw CacheError("request already holds cache");
  const auto need = needs(total_tokens);
  bool ok = state_slots_ == 0 || !free_slots_.empty();
  for (int g = 0; ok && g < num_groups(); ++g) ok = need[g] <= pools_[g].available();
  if (!ok) {
    ++allocation_failures_;
    return false;
  }
  Entry e;
  e.tables.resize(groups_.size());
  e.trimmed.assign(groups_.size(), 0);
  e.reserved = need;
  e.has_reservation = true;
  for (int g = 0; g < num_groups(); ++g) pools_[g].reserve(need[g]);
  if (state_slots_ > 0) {
    e.slot = free_slots_.back();
    free_slots_.pop_back();
    slots_to_clear_.push_back(e.slot);
  }
  requests_.emplace(id, std::move(e));
  return true;
}

void CacheManager::open(RequestId id) {
  if (contains(id)) throw CacheError("request already holds cache");
  Entry e;
  e.tables.resize(groups_.size());
  e.trimmed.assign(groups_.size(), 0);
  e.reserved.assign(groups_.size(), 0);
  if (state_slots_ > 0) {
    if (free_slots_.empty()) throw CacheError("no state slot is free");
    e.slot = free_slots_.back();
    free_slots_.pop_back();
    slots_to_clear_.push_back(e.slot);
  }
  requests_.emplace(id, std::move(e));
}

CacheManager::Entry& CacheManager::entry(RequestId id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) throw CacheError("request holds no cache");
  return it->second;
}
const CacheManager::Entry& CacheManager::entry(RequestId id) const {
  auto it = requests_.find(id);
  if (it == requests_.end()) throw CacheError("request holds no cache");
  return it->second;
}

int CacheManager::take_page(Entry& e, int g) {
  if (e.reserved[g] > 0) {
    --e.reserved[g];
    return pools_[g].allocate(true);
  }
  if (e.has_reservation && !groups_[g].window)
    throw CacheError("request exceeded its K/V reservation");
  if (pools_[g].available() <= 0) {
    ++allocation_failures_;
    throw CacheError("the K/V page pool of group '" + groups_[g].name + "' is exhausted");
  }
  return pools_[g].allocate(false);
}

void CacheManager::ensure(RequestId id, int end) {
  Entry& e = entry(id);
  if (end < e.length) throw CacheError("K/V token count cannot shrink");
  for (int g = 0; g < num_groups(); ++g) {
    auto& table = e.tables[g];
    while (static_cast<std::int64_t>(table.size()) * page_size_ < end)
      table.push_back(take_page(e, g));
  }
}

void CacheManager::advance(RequestId id, int length) {
  Entry& e = entry(id);
  if (length < e.length) throw CacheError("K/V token count cannot shrink");
  for (int g = 0; g < num_groups(); ++g)
    if (static_cast<std::int64_t>(e.tables[g].size()) * page_size_ < length)
      throw CacheError("advanced past the pages the request holds");
  e.length = length;
  for (int g = 0; g < num_groups(); ++g) {
    const int window = groups_[g].window;
    if (!window) continue;
    auto& table = e.tables[g];
    // The next position is `length`; it sees positions > length - window.
    const int first_live_position = std::max(0, length - window + 1);
    const int first_live = std::min(static_cast<int>(table.size()), first_live_position / page_size_);
    for (int index = e.trimmed[g]; index < first_live; ++index) {
      const int page = table[index];
      if (page < 0) continue;
      pools_[g].release(page);
      table[index] = -1;
      // Keep the quota: the window moves on and will need a page.
      if (e.has_reservation && pools_[g].reserve(1)) ++e.reserved[g];
    }
    e.trimmed[g] = std::max(e.trimmed[g], first_live);
  }
}

void CacheManager::release(RequestId id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return;
  Entry& e = it->second;
  for (int g = 0; g < num_groups(); ++g) {
    for (int page : e.tables[g])
      if (page >= 0) pools_[g].release(page);
    pools_[g].unreserve(e.reserved[g]);
  }
  if (e.slot >= 0) free_slots_.push_back(e.slot);
  requests_.erase(it);
}

const std::vector<int>& CacheManager::table(RequestId id, int g) const {
  return entry(id).tables.at(g);
}
int CacheManager::slot(RequestId id) const { return entry(id).slot; }
int CacheManager::length(RequestId id) const { return entry(id).length; }

std::vector<int> CacheManager::take_slots_to_clear() {
  std::vector<int> out;
  out.swap(slots_to_clear_);
  return out;
}

void CacheManager::fill_tables(const std::vector<RequestId>& ids, int g, std::int32_t* out,
                               int stride, std::int32_t pad) const {
  for (std::size_t i = 0; i < ids.size(); ++i) {
    const auto& table = entry(ids[i]).tables.at(g);
    if (static_cast<int>(table.size()) > stride)
      throw CacheError("a block table is longer than the device table's row");
    std::int32_t* row = out + i * static_cast<std::size_t>(stride);
    for (int p = 0; p < stride; ++p)
      row[p] = p < static_cast<int>(table.size()) ? table[p] : pad;
  }
}

CacheStats CacheManager::stats() const {
  CacheStats out;
  for (int g = 0; g < num_groups(); ++g) {
    GroupStats s;
    s.name = groups_[g].name;
    s.window = groups_[g].window;
    s.capacity_pages = pools_[g].capacity();
    s.used_pages = pools_[g].used();
    s.reserved_pages = pools_[g].reserved();
    s.free_pages = pools_[g].free_pages();
    s.high_water = pools_[g].high_water();
    out.groups.push_back(s);
  }
  for (const auto& [id, e] : requests_) {
    (void)id;
    out.live_tokens += e.length;
    if (!e.tables.empty() && !e.tables[0].empty()) {
      std::int64_t held = 0;
      for (int page : e.tables[0]) held += page >= 0 ? page_size_ : 0;
      const int window = groups_[0].window;
      const std::int64_t live = window ? std::min(e.length, window) : e.length;
      out.internal_fragmentation_tokens += std::max<std::int64_t>(0, held - live);
    }
  }
  out.allocation_failures = allocation_failures_;
  out.state_slots = state_slots_;
  out.free_state_slots = static_cast<int>(free_slots_.size());
  out.requests = static_cast<int>(requests_.size());
  return out;
}

void CacheManager::check_invariants() const {
  for (int g = 0; g < num_groups(); ++g) {
    const PagePool& pool = pools_[g];
    std::vector<int> holders(pool.capacity(), 0);
    int reserved = 0;
    for (const auto& [id, e] : requests_) {
      (void)id;
      reserved += e.reserved[g];
      for (int page : e.tables[g]) {
        if (page < 0) continue;
        if (page >= pool.capacity()) throw CacheError("a table names a page past the pool");
        ++holders[page];
      }
    }
    int held = 0;
    for (int page = 0; page < pool.capacity(); ++page) {
      if (holders[page] != pool.refcount(page))
        throw CacheError("page " + std::to_string(page) + " of group '" + groups_[g].name +
                         "' has " + std::to_string(pool.refcount(page)) + " holders recorded but " +
                         std::to_string(holders[page]) + " tables name it");
      if (holders[page] > 1) throw CacheError("a page is held twice");
      held += holders[page] ? 1 : 0;
    }
    if (held != pool.used()) throw CacheError("used-page count disagrees with the tables (a page was lost)");
    if (reserved != pool.reserved()) throw CacheError("reserved-page count disagrees with the requests");
    if (pool.reserved() > pool.free_pages()) throw CacheError("more pages promised than free");
  }
  std::set<int> slots(free_slots_.begin(), free_slots_.end());
  if (slots.size() != free_slots_.size()) throw CacheError("a state slot is free twice");
  for (const auto& [id, e] : requests_) {
    (void)id;
    if (e.slot >= 0 && !slots.insert(e.slot).second) throw CacheError("a state slot is held twice");
  }
  if (static_cast<int>(slots.size()) != state_slots_) throw CacheError("a state slot was lost");
}

}  // namespace b200
