// Continuous-batching scheduler: admission, the plan of one step, and what follows a step.
//
// Requests wait first-come-first-served until a sequence slot and the pages for their whole
// budget (prompt + max_new_tokens) can be promised (python/instinct/mlx_engine.py:272-297).
// A step's plan holds one token for every running request, then portions of admitted
// prompts, each at most `prefill_chunk_size` tokens, while the step's token budget lasts;
// the reference runs decode and one prompt chunk as two passes per step
// (mlx_engine.py:404-453), here they are one batch. After the step the sampled tokens are
// committed: a request finishes on a stop token, at its token budget, or at the context
// limit (mlx_engine.py:511-527), and its pages return to the pools.
// Pages cannot run out mid-request because admission reserved them; a request that could
// never fit is refused at submit (mlx_engine.py:227-229), one that does not fit now waits.
#pragma once

#include <cstdint>
#include <deque>
#include <optional>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "cache_manager.h"

namespace b200 {

enum class SequenceState : std::uint8_t { waiting, prefilling, running, completed, cancelled, rejected };

// One row of the table of allowed sampling settings (field, interval, whether whole numbers only).
struct SamplingRange {
  const char* field;
  double low, high;
  bool low_open, high_open, whole;
};
const std::vector<SamplingRange>& sampling_ranges();

struct SamplingParams {
  double temperature{0.0};
  double top_p{1.0};
  int top_k{0};
  double min_p{0.0};
  std::optional<std::int64_t> seed;

  void validate() const;
  bool greedy() const { return temperature == 0.0 || top_k == 1; }
};

struct Request {
  RequestId id{};
  SequenceState state{SequenceState::waiting};
  std::vector<std::int32_t> prompt;
  std::vector<std::int32_t> output;
  std::unordered_set<std::int32_t> stop;
  int max_new_tokens{0};
  SamplingParams sampling;
  std::int64_t seed{0};  // the request's own or one drawn from the scheduler's stream
  std::string reason;
  int length{0};  // positions whose keys and values are in the cache
  std::deque<std::int32_t> forced;
};

struct PlanEntry {
  RequestId id{};
  int start{0};          // position of the entry's first token
  int count{0};          // tokens fed this step
  int token_offset{0};   // into Plan::tokens
  bool decode{false};
  bool wants_token{false};  // the step's last logits of this entry choose a token
};

struct Plan {
  std::vector<PlanEntry> entries;
  std::vector<std::int32_t> tokens;  // all entries' tokens, in entry order
  int total_tokens() const { return static_cast<int>(tokens.size()); }
};

struct TokenEvent {
  RequestId request_id{};
  std::int32_t token{};
  bool finished{false};
  std::string reason;
};

struct SchedulerStats {
  std::uint64_t submitted{}, completed{}, cancelled{}, rejected{};
  std::uint64_t prompt_tokens{}, generated_tokens{}, steps{};
  std::uint32_t waiting{}, running{};
};

class Scheduler {
 public:
  // A prompt portion is at most `prefill_chunk_size` tokens while anything is decoding and at
  // most `prefill_burst_size` when nothing is (python/instinct/mlx_engine.py:430).
  Scheduler(CacheManager& cache, int max_num_sequences, int max_model_length,
            int max_batch_tokens, int prefill_chunk_size, int prefill_burst_size, int vocab_size,
            std::uint64_t seed);

  RequestId submit(std::vector<std::int32_t> prompt, int max_new_tokens,
                   const std::vector<std::int32_t>& stop, const SamplingParams& sampling);
  void force(RequestId id, const std::vector<std::int32_t>& tokens);
  void cancel(RequestId id);
  void forget(RequestId id);
  const Request& request(RequestId id) const;
  bool has_work() const { return !waiting_.empty() || !running_.empty(); }

  // Admit what fits, then lay out the next step. The plan may be empty.
  Plan plan();
  // `tokens[i]` is the token chosen for the i-th entry with wants_token, in entry order.
  std::vector<TokenEvent> commit(const Plan& plan, const std::vector<std::int32_t>& tokens);
  // The step threw: every request it held is cancelled with reason "error".
  void abandon(const Plan& plan);

  // Key of the uniform draw for the request's next token: (seed * 1000003 + generated) mod 2^63
  // (python/instinct/sampling.py:94-98).
  std::uint64_t draw_key(RequestId id) const;
  // True when the step after `plan` is bound to feed the same requests one token each, unless
  // a token sampled in this step ends one of them: every entry is a running request's single
  // token, no request waits for admission or is still reading its prompt, none reaches its
  // length or context limit with this step's token, and none has a forced token pending.
  // The engine may then launch that next step before it has read this step's tokens.
  bool repeats(const Plan& plan) const;

  SchedulerStats stats() const;
  int max_model_length() const { return max_model_length_; }

 private:
  Request& mutable_request(RequestId id);
  void finish(Request& request, SequenceState state, const std::string& reason);
  void admit();

  CacheManager& cache_;
  int max_num_sequences_, max_model_length_, max_batch_tokens_, prefill_chunk_size_,
      prefill_burst_size_, vocab_size_;
  std::uint64_t seed_stream_;
  RequestId next_id_{1};
  std::deque<RequestId> waiting_;
  std::vector<RequestId> running_;
  std::unordered_map<RequestId, Request> requests_;
  SchedulerStats totals_{};
};

}  // namespace b200
