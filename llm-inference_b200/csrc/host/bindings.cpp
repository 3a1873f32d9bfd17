// pybind11 surface of the host runtime: page pools, the cache manager and the scheduler.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace b200;

namespace {

const char* state_name(SequenceState s) {
  switch (s) {
    case SequenceState::waiting: return "waiting";
    case SequenceState::prefilling: return "prefilling";
    case SequenceState::running: return "running";
    case SequenceState::completed: return "completed";
    case SequenceState::cancelled: return "cancelled";
    case SequenceState::rejected: return "rejected";
  }
  return "?";
}

template <typename T>
py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> out(static_cast<py::ssize_t>(v.size()));
  std::copy(v.begin(), v.end(), out.mutable_data());
  return out;
}

}  // namespace

PYBIND11_MODULE(b200_host, m) {
  m.doc() = "Host runtime of the engine: paged-cache bookkeeping and the continuous-batching scheduler";
  py::register_exception<CacheError>(m, "CacheError", PyExc_RuntimeError);

  py::class_<PagePool>(m, "PagePool")
      .def(py::init<int>(), py::arg("capacity"))
      .def_property_readonly("capacity", &PagePool::capacity)
      .def_property_readonly("free", &PagePool::free_pages)
      .def_property_readonly("available", &PagePool::available)
      .def_property_readonly("used", &PagePool::used)
      .def_property_readonly("reserved", &PagePool::reserved)
      .def_property_readonly("high_water", &PagePool::high_water)
      .def("reserve", &PagePool::reserve)
      .def("unreserve", &PagePool::unreserve)
      .def("allocate", &PagePool::allocate, py::arg("reserved"))
      .def("retain", &PagePool::retain)
      .def("release", &PagePool::release)
      .def("refcount", &PagePool::refcount);

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](std::string name, int capacity_pages, int window) {
             return GroupSpec{std::move(name), capacity_pages, window};
           }),
           py::arg("name"), py::arg("capacity_pages"), py::arg("window") = 0)
      .def_readwrite("name", &GroupSpec::name)
      .def_readwrite("capacity_pages", &GroupSpec::capacity_pages)
      .def_readwrite("window", &GroupSpec::window);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<int, std::vector<GroupSpec>, int, int>(), py::arg("page_size"), py::arg("groups"),
           py::arg("state_slots"), py::arg("step_tokens"))
      .def_property_readonly("page_size", &CacheManager::page_size)
      .def_property_readonly("num_groups", &CacheManager::num_groups)
      .def("group", &CacheManager::group)
      .def("group_index", &CacheManager::group_index)
      .def("needs", &CacheManager::needs)
      .def("can_ever_fit", &CacheManager::can_ever_fit)
      .def("admit", &CacheManager::admit)
      .def("open", &CacheManager::open)
      .def("contains", &CacheManager::contains)
      .def("ensure", &CacheManager::ensure)
      .def("advance", &CacheManager::advance)
      .def("release", &CacheManager::release)
      .def("table", [](const CacheManager& c, RequestId id, int g) { return c.table(id, g); })
      .def("slot", &CacheManager::slot)
      .def("length", &CacheManager::length)
      .def("take_slots_to_clear", &CacheManager::take_slots_to_clear)
      .def("fill_tables",
           [](const CacheManager& c, const std::vector<RequestId>& ids, int g,
              py::array_t<std::int32_t, py::array::c_style> out, std::int32_t pad) {
             if (out.ndim() != 2 || out.shape(0) < static_cast<py::ssize_t>(ids.size()))
               throw std::invalid_argument("fill_tables needs a [requests, pages] int32 array");
             c.fill_tables(ids, g, out.mutable_data(), static_cast<int>(out.shape(1)), pad);
           },
           py::arg("ids"), py::arg("group"), py::arg("out"), py::arg("pad") = 0)
      .def("count_allocation_failure", &CacheManager::count_allocation_failure)
      .def("check_invariants", &CacheManager::check_invariants)
      .def("stats", [](const CacheManager& c) {
        const CacheStats s = c.stats();
        py::dict groups;
        for (const auto& g : s.groups) {
          py::dict d;
          d["window"] = g.window;
          d["capacity_pages"] = g.capacity_pages;
          d["used_pages"] = g.used_pages;
          d["reserved_pages"] = g.reserved_pages;
          d["free_pages"] = g.free_pages;
          d["high_water"] = g.high_water;
          groups[py::str(g.name)] = d;
        }
        py::dict out;
        out["kv_pools"] = groups;
        out["live_tokens"] = s.live_tokens;
        out["internal_fragmentation_tokens"] = s.internal_fragmentation_tokens;
        out["allocation_failures"] = s.allocation_failures;
        out["state_slots"] = s.state_slots;
        out["free_state_slots"] = s.free_state_slots;
        out["requests"] = s.requests;
        return out;
      });

  m.def("sampling_ranges", []() {
    py::dict out;
    for (const SamplingRange& r : sampling_ranges())
      out[r.field] = py::make_tuple(r.low, r.high, r.low_open, r.high_open, r.whole);
    return out;
  });

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init([](double temperature, double top_p, int top_k, double min_p,
                       std::optional<std::int64_t> seed) {
             SamplingParams p{temperature, top_p, top_k, min_p, seed};
             p.validate();
             return p;
           }),
           py::arg("temperature") = 0.0, py::arg("top_p") = 1.0, py::arg("top_k") = 0,
           py::arg("min_p") = 0.0, py::arg("seed") = py::none())
      .def_readonly("temperature", &SamplingParams::temperature)
      .def_readonly("top_p", &SamplingParams::top_p)
      .def_readonly("top_k", &SamplingParams::top_k)
      .def_readonly("min_p", &SamplingParams::min_p)
      .def_readonly("seed", &SamplingParams::seed)
      .def_property_readonly("greedy", &SamplingParams::greedy);

  py::class_<Request>(m, "Request")
      .def_readonly("request_id", &Request::id)
      .def_property_readonly("state", [](const Request& r) { return std::string(state_name(r.state)); })
      .def_property_readonly("prompt", [](const Request& r) { return to_array(r.prompt); })
      .def_property_readonly("output", [](const Request& r) { return r.output; })
      .def_readonly("max_new_tokens", &Request::max_new_tokens)
      .def_readonly("sampling", &Request::sampling)
      .def_readonly("seed", &Request::seed)
      .def_readonly("reason", &Request::reason)
      .def_readonly("length", &Request::length);

  py::class_<PlanEntry>(m, "PlanEntry")
      .def_readonly("request_id", &PlanEntry::id)
      .def_readonly("start", &PlanEntry::start)
      .def_readonly("count", &PlanEntry::count)
      .def_readonly("token_offset", &PlanEntry::token_offset)
      .def_readonly("decode", &PlanEntry::decode)
      .def_readonly("wants_token", &PlanEntry::wants_token);

  py::class_<Plan>(m, "Plan")
      .def_readonly("entries", &Plan::entries)
      .def_property_readonly("tokens", [](const Plan& p) { return to_array(p.tokens); })
      .def_property_readonly("total_tokens", &Plan::total_tokens)
      .def_property_readonly("ids",
                             [](const Plan& p) {
                               std::vector<RequestId> v;
                               for (const auto& e : p.entries) v.push_back(e.id);
                               return v;
                             })
      .def_property_readonly("starts",
                             [](const Plan& p) {
                               std::vector<std::int32_t> v;
                               for (const auto& e : p.entries) v.push_back(e.start);
                               return to_array(v);
                             })
      .def_property_readonly("counts",
                             [](const Plan& p) {
                               std::vector<std::int32_t> v;
                               for (const auto& e : p.entries) v.push_back(e.count);
                               return to_array(v);
                             })
      .def_property_readonly("wanting", [](const Plan& p) {
        std::vector<std::int32_t> v;
        for (std::size_t i = 0; i < p.entries.size(); ++i)
          if (p.entries[i].wants_token) v.push_back(static_cast<std::int32_t>(i));
        return v;
      });

  py::class_<TokenEvent>(m, "TokenEvent")
      .def_readonly("request_id", &TokenEvent::request_id)
      .def_readonly("token", &TokenEvent::token)
      .def_readonly("finished", &TokenEvent::finished)
      .def_readonly("reason", &TokenEvent::reason)
      .def("__repr__", [](const TokenEvent& e) {
        return "TokenEvent(request_id=" + std::to_string(e.request_id) + ", token=" +
               std::to_string(e.token) + ", finished=" + (e.finished ? "True" : "False") +
               ", reason='" + e.reason + "')";
      });

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<CacheManager&, int, int, int, int, int, int, std::uint64_t>(), py::arg("cache"),
           py::arg("max_num_sequences"), py::arg("max_model_length"), py::arg("max_batch_tokens"),
           py::arg("prefill_chunk_size"), py::arg("prefill_burst_size"), py::arg("vocab_size"),
           py::arg("seed") = 0,
           py::keep_alive<1, 2>())
      .def("submit", &Scheduler::submit, py::arg("prompt"), py::arg("max_new_tokens"),
           py::arg("stop") = std::vector<std::int32_t>{}, py::arg("sampling") = SamplingParams{})
      .def("force", &Scheduler::force)
      .def("cancel", &Scheduler::cancel)
      .def("forget", &Scheduler::forget)
      .def("request", &Scheduler::request, py::return_value_policy::reference_internal)
      .def("has_work", &Scheduler::has_work)
      .def("plan", &Scheduler::plan)
      .def("commit", &Scheduler::commit)
      .def("abandon", &Scheduler::abandon)
      .def("draw_key", &Scheduler::draw_key)
      .def("repeats", &Scheduler::repeats)
      .def_property_readonly("max_model_length", &Scheduler::max_model_length)
      .def("stats", [](const Scheduler& s) {
        const SchedulerStats t = s.stats();
        py::dict out;
        out["submitted"] = t.submitted;
        out["completed"] = t.completed;
        out["cancelled"] = t.cancelled;
        out["rejected"] = t.rejected;
        out["prompt_tokens"] = t.prompt_tokens;
        out["generated_tokens"] = t.generated_tokens;
        out["steps"] = t.steps;
        out["waiting"] = t.waiting;
        out["running"] = t.running;
        return out;
      });
}
