#include "scheduler.h"

#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace b200 {

const std::vector<SamplingRange>& sampling_ranges() {
  // The same table as sampling/params.py::RANGES; a test compares them.
  static const std::vector<SamplingRange> table = {
      {"temperature", 0.0, 10.0, false, false, false},
      {"top_p", 0.0, 1.0, true, false, false},
      {"top_k", 0.0, 2147483647.0, false, false, true},
      {"min_p", 0.0, 1.0, false, true, false},
  };
  return table;
}

void SamplingParams::validate() const {
  const double values[] = {temperature, top_p, static_cast<double>(top_k), min_p};
  std::string broken;
  std::size_t i = 0;
  for (const SamplingRange& r : sampling_ranges()) {
    const double v = values[i++];
    const bool above = r.low_open ? v > r.low : v >= r.low;
    const bool below = r.high_open ? v < r.high : v <= r.high;
    if (std::isfinite(v) && above && below) continue;
    if (!broken.empty()) broken += "; ";
    broken += std::string(r.field) + "=" + std::to_string(v) + " is outside " + (r.low_open ? "(" : "[") +
              std::to_string(r.low) + ", " + std::to_string(r.high) + (r.high_open ? ")" : "]");
  }
  if (!broken.empty()) throw std::invalid_argument("sampling settings refused: " + broken);
}

Scheduler::Scheduler(CacheManager& cache, int max_num_sequences, int max_model_length,
                     int max_batch_tokens, int prefill_chunk_size, int prefill_burst_size,
                     int vocab_size, std::uint64_t seed)
    : cache_(cache), max_num_sequences_(max_num_sequences), max_model_length_(max_model_length),
      max_batch_tokens_(max_batch_tokens), prefill_chunk_size_(prefill_chunk_size),
      prefill_burst_size_(prefill_burst_size), vocab_size_(vocab_size), seed_stream_(seed) {
  if (max_num_sequences <= 0 || max_model_length <= 0)
    throw std::invalid_argument("sequence and context limits must be positive");
  if (prefill_chunk_size <= 0 || prefill_burst_size < prefill_chunk_size)
    throw std::invalid_argument("prefill chunk sizes must be positive, the burst no smaller");
  if (max_batch_tokens < max_num_sequences)
    throw std::invalid_argument("max_batch_tokens must allow one token per sequence");
  if (vocab_size <= 0) throw std::invalid_argument("vocabulary size must be positive");
}

RequestId Scheduler::submit(std::vector<std::int32_t> prompt, int max_new_tokens,
                            const std::vector<std::int32_t>& stop, const SamplingParams& sampling) {
  sampling.validate();
  if (prompt.empty()) throw std::invalid_argument("the prompt must be a non-empty list of token ids");
  for (auto t : prompt)
    if (t < 0 || t >= vocab_size_) throw std::invalid_argument("token id is outside the vocabulary");
  for (auto t : stop)
    if (t < 0 || t >= vocab_size_) throw std::invalid_argument("token id is outside the vocabulary");
  if (max_new_tokens <= 0) throw std::invalid_argument("max_new_tokens must be a positive integer");
  const std::int64_t total = static_cast<std::int64_t>(prompt.size()) + max_new_tokens;
  if (total > max_model_length_)
    throw std::invalid_argument(std::to_string(prompt.size()) + " prompt tokens plus " +
                                std::to_string(max_new_tokens) + " new ones exceed the " +
                                std::to_string(max_model_length_) + "-token context");
  if (!cache_.can_ever_fit(static_cast<int>(total))) {
    ++totals_.rejected;
    throw std::invalid_argument("the request needs more K/V memory than the cache has");
  }
  Request r;
  r.id = next_id_++;
  r.prompt = std::move(prompt);
  r.max_new_tokens = max_new_tokens;
  r.stop.insert(stop.begin(), stop.end());
  r.sampling = sampling;
  if (sampling.seed) {
    r.seed = *sampling.seed;
  } else {
    // splitmix64 step over the scheduler's own stream
    seed_stream_ += 0x9E3779B97F4A7C15ull;
    std::uint64_t z = seed_stream_;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    r.seed = static_cast<std::int64_t>((z ^ (z >> 31)) >> 2);
  }
  const RequestId id = r.id;
  requests_.emplace(id, std::move(r));
  waiting_.push_back(id);
  ++totals_.submitted;
  return id;
}

void Scheduler::force(RequestId id, const std::vector<std::int32_t>& tokens) {
  auto& r = mutable_request(id);
  for (auto t : tokens) {
    if (t < 0 || t >= vocab_size_) throw std::invalid_argument("token id is outside the vocabulary");
    r.forced.push_back(t);
  }
}

Request& Scheduler::mutable_request(RequestId id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) throw std::out_of_range("unknown request id");
  return it->second;
}

const Request& Scheduler::request(RequestId id) const {
  auto it = requests_.find(id);
  if (it == requests_.end()) throw std::out_of_range("unknown request id");
  return it->second;
}

void Scheduler::finish(Request& r, SequenceState state, const std::string& reason) {
  running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
  cache_.release(r.id);
  r.state = state;
  r.reason = reason;
  if (state == SequenceState::completed) ++totals_.completed;
  else ++totals_.cancelled;
}

void Scheduler::cancel(RequestId id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return;
  Request& r = it->second;
  if (r.state == SequenceState::completed || r.state == SequenceState::cancelled ||
      r.state == SequenceState::rejected)
    return;
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  finish(r, SequenceState::cancelled, "cancelled");
}

void Scheduler::forget(RequestId id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return;
  const auto state = it->second.state;
  if (state == SequenceState::waiting || state == SequenceState::prefilling ||
      state == SequenceState::running)
    throw std::runtime_error("cannot forget an active request");
  requests_.erase(it);
}

void Scheduler::admit() {
  while (!waiting_.empty() && static_cast<int>(running_.size()) < max_num_sequences_) {
    Request& r = mutable_request(waiting_.front());
    const int total = static_cast<int>(r.prompt.size()) + r.max_new_tokens;
    if (!cache_.admit(r.id, total)) return;  // head of the line waits; nobody overtakes it
    waiting_.pop_front();
    r.state = SequenceState::prefilling;
    running_.push_back(r.id);
    totals_.prompt_tokens += r.prompt.size();
  }
}

Plan Scheduler::plan() {
  admit();
  Plan plan;
  int budget = max_batch_tokens_;
  for (RequestId id : running_) {
    Request& r = mutable_request(id);
    if (r.state != SequenceState::running) continue;
    PlanEntry e;
    e.id = id;
    e.start = r.length;
    e.count = 1;
    e.token_offset = plan.total_tokens();
    e.decode = true;
    e.wants_token = true;
    plan.tokens.push_back(r.output.back());
    plan.entries.push_back(e);
    --budget;
  }
  const int portion = plan.entries.empty() ? prefill_burst_size_ : prefill_chunk_size_;
  for (RequestId id : running_) {
    if (budget <= 0) break;
    Request& r = mutable_request(id);
    if (r.state != SequenceState::prefilling) continue;
    const int remaining = static_cast<int>(r.prompt.size()) - r.length;
    const int count = std::min({remaining, portion, budget});
    PlanEntry e;
    e.id = id;
    e.start = r.length;
    e.count = count;
    e.token_offset = plan.total_tokens();
    e.decode = false;
    e.wants_token = (count == remaining);
    plan.tokens.insert(plan.tokens.end(), r.prompt.begin() + r.length,
                       r.prompt.begin() + r.length + count);
    plan.entries.push_back(e);
    budget -= count;
  }
  for (const auto& e : plan.entries) cache_.ensure(e.id, e.start + e.count);
  return plan;
}

std::vector<TokenEvent> Scheduler::commit(const Plan& plan, const std::vector<std::int32_t>& tokens) {
  std::size_t wanted = 0;
  for (const auto& e : plan.entries) wanted += e.wants_token ? 1 : 0;
  if (wanted != tokens.size()) throw std::invalid_argument("commit needs one token per wanting entry");
  std::vector<TokenEvent> events;
  std::size_t next = 0;
  for (const auto& e : plan.entries) {
    auto it = requests_.find(e.id);
    const bool alive = it != requests_.end() && (it->second.state == SequenceState::prefilling ||
                                                 it->second.state == SequenceState::running);
    std::int32_t token = e.wants_token ? tokens[next++] : -1;
    if (!alive) continue;  // cancelled while the step ran
    Request& r = it->second;
    r.length = e.start + e.count;
    cache_.advance(r.id, r.length);
    if (!e.wants_token) continue;
    if (!r.forced.empty()) {
      token = r.forced.front();
      r.forced.pop_front();
    }
    if (token < 0 || token >= vocab_size_) throw std::invalid_argument("sampled token is outside the vocabulary");
    r.state = SequenceState::running;
    r.output.push_back(token);
    ++totals_.generated_tokens;
    std::string reason;
    if (r.stop.count(token)) reason = "stop";
    else if (static_cast<int>(r.output.size()) >= r.max_new_tokens) reason = "length";
    else if (r.length + 1 >= max_model_length_) reason = "context";
    if (!reason.empty()) finish(r, SequenceState::completed, reason);
    events.push_back(TokenEvent{r.id, token, !reason.empty(), reason});
  }
  ++totals_.steps;
  return events;
}

void Scheduler::abandon(const Plan& plan) {
  for (const auto& e : plan.entries) {
    auto it = requests_.find(e.id);
    if (it == requests_.end()) continue;
    Request& r = it->second;
    if (r.state == SequenceState::prefilling || r.state == SequenceState::running)
      finish(r, SequenceState::cancelled, "error");
  }
}

bool Scheduler::repeats(const Plan& plan) const {
  if (plan.entries.empty() || !waiting_.empty() || plan.entries.size() != running_.size()) return false;
  for (const auto& e : plan.entries) {
    if (!e.decode || e.count != 1 || !e.wants_token) return false;
    auto it = requests_.find(e.id);
    if (it == requests_.end()) return false;
    const Request& r = it->second;
    if (r.state != SequenceState::running || !r.forced.empty()) return false;
    if (static_cast<int>(r.output.size()) + 1 >= r.max_new_tokens) return false;  // ends by length
    if (e.start + 2 >= max_model_length_) return false;                           // ends by context
  }
  return true;
}

std::uint64_t Scheduler::draw_key(RequestId id) const {
  const Request& r = request(id);
  const __int128 modulus = static_cast<__int128>(1) << 63;
  __int128 wide = static_cast<__int128>(r.seed) * 1000003 + static_cast<__int128>(r.output.size());
  wide %= modulus;
  if (wide < 0) wide += modulus;
  return static_cast<std::uint64_t>(wide);
}

SchedulerStats Scheduler::stats() const {
  SchedulerStats out = totals_;
  out.waiting = static_cast<std::uint32_t>(waiting_.size());
  out.running = static_cast<std::uint32_t>(running_.size());
  return out;
}

}  // namespace b200
