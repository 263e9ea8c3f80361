#include "batch_scheduler.hpp"

#include <algorithm>
#include <chrono>
#include <stdexcept>

namespace pocket {

double BatchScheduler::now() {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}

BatchScheduler::BatchScheduler(InferenceEngine& engine, SchedulerOptions options) : BatchScheduler(engine, options, true) {}

BatchScheduler::BatchScheduler(InferenceEngine& engine, SchedulerOptions options, bool start_thread)
    : eng_(engine), opt_(options) {
  if (opt_.max_batch < 1 || opt_.prefill_token_budget < 1 || opt_.prefill_chunk_tokens < 1)
    throw std::invalid_argument("BatchScheduler: options must be positive");
  opt_.max_batch = std::min(opt_.max_batch, eng_.max_slots());
  stats_.kv_blocks_total = eng_.total_blocks();
  if (start_thread) thread_ = std::thread([this] { loop(); });
}

std::unique_ptr<BatchScheduler> BatchScheduler::make_manual(InferenceEngine& engine, SchedulerOptions options) {
  return std::unique_ptr<BatchScheduler>(new BatchScheduler(engine, options, false));
}

BatchScheduler::~BatchScheduler() { stop(); }

void BatchScheduler::stop() {
  bool was = stop_.exchange(true);
  cv_work_.notify_all();
  if (thread_.joinable()) thread_.join();
  if (was) return;
  std::lock_guard<std::mutex> g(mu_);
  auto drain = [&](std::unique_ptr<Seq> s) { finish(std::move(s), "cancelled"); };
  while (!queue_.empty()) { auto s = std::move(queue_.front()); queue_.pop_front(); drain(std::move(s)); }
  for (auto& s : prefilling_) drain(std::move(s));
  for (auto& s : decoding_) drain(std::move(s));
  prefilling_.clear();
  decoding_.clear();
  cv_done_.notify_all();
}

uint64_t BatchScheduler::submit(std::vector<int32_t> prompt, int max_new_tokens, bool stop_on_eos) {
  if (prompt.empty()) throw std::invalid_argument("submit: empty prompt");
  if (max_new_tokens < 1) throw std::invalid_argument("submit: max_new_tokens must be >= 1");
  if (static_cast<int64_t>(prompt.size()) + max_new_tokens > eng_.max_context())
    throw std::invalid_argument("submit: prompt + max_new_tokens exceeds the engine's context");
  if (stop_.load()) throw std::runtime_error("submit: scheduler stopped");
  auto s = std::make_unique<Seq>();
  s->req.prompt = std::move(prompt);
  s->req.max_new_tokens = max_new_tokens;
  s->req.stop_on_eos = stop_on_eos;
  s->t_submit = now();
  std::lock_guard<std::mutex> g(mu_);
  s->req.id = next_id_++;
  // a request that could never fit even in an empty pool is refused now instead of blocking the queue forever
  if (worst_case_blocks(*s) > eng_.total_blocks()) throw std::invalid_argument("submit: request needs more KV blocks than the pool has");
  const uint64_t id = s->req.id;
  queue_.push_back(std::move(s));
  stats_.queued = static_cast<int>(queue_.size());
  cv_work_.notify_one();
  return id;
}

bool BatchScheduler::cancel(uint64_t id) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto it = queue_.begin(); it != queue_.end(); ++it)
    if ((*it)->req.id == id) {
      auto s = std::move(*it);
      queue_.erase(it);
      finish(std::move(s), "cancelled");
      cv_done_.notify_all();
      return true;
    }
  for (auto* vec : {&prefilling_, &decoding_})
    for (auto& s : *vec)
      if (s->req.id == id) { s->cancelled = true; cv_work_.notify_one(); return true; }
  return false;
}

bool BatchScheduler::poll(uint64_t id, SchedulerResult& out) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = done_.find(id);
  if (it == done_.end()) return false;
  out = std::move(it->second);
  done_.erase(it);
  return true;
}

bool BatchScheduler::wait(uint64_t id, SchedulerResult& out, int timeout_ms) {
  std::unique_lock<std::mutex> g(mu_);
  auto ready = [&] { return done_.count(id) != 0; };
  if (timeout_ms < 0) cv_done_.wait(g, ready);
  else if (!cv_done_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready)) return false;
  auto it = done_.find(id);
  out = std::move(it->second);
  done_.erase(it);
  return true;
}

SchedulerStats BatchScheduler::stats() const {
  std::lock_guard<std::mutex> g(mu_);
  SchedulerStats s = stats_;
  s.queued = static_cast<int>(queue_.size());
  s.prefilling = static_cast<int>(prefilling_.size());
  s.decoding = static_cast<int>(decoding_.size());
  s.kv_blocks_reserved = reserved_blocks_;
  return s;
}

int BatchScheduler::worst_case_blocks(const Seq& s) const {
  const int64_t tokens = static_cast<int64_t>(s.req.prompt.size()) + s.req.max_new_tokens;
  const int bt = eng_.block_tokens();
  return static_cast<int>((tokens + bt - 1) / bt);
}

// mu_ held by the caller
void BatchScheduler::finish(std::unique_ptr<Seq> s, const char* reason, const std::string& error) {
  if (s->slot >= 0) eng_.free_slot(s->slot);
  reserved_blocks_ -= s->reserved_blocks;
  SchedulerResult r;
  r.id = s->req.id;
  r.tokens = std::move(s->out);
  r.finish_reason = reason;
  r.error = error;
  const double t = now();
  r.queue_seconds = (s->t_admit > 0 ? s->t_admit : t) - s->t_submit;
  r.prefill_seconds = s->t_first > 0 ? s->t_first - s->t_admit : 0;
  r.decode_seconds = s->t_first > 0 ? t - s->t_first : 0;
  if (std::string(reason) == "cancelled") ++stats_.cancelled;
  else if (std::string(reason) == "error") ++stats_.failed;
  else ++stats_.completed;
  done_[r.id] = std::move(r);
}

// mu_ held
void BatchScheduler::admit() {
  while (!queue_.empty()) {
    if (static_cast<int>(prefilling_.size() + decoding_.size()) >= opt_.max_batch) return;
    Seq& head = *queue_.front();
    const int need = worst_case_blocks(head);
    // head-of-line blocking: a later, smaller request never jumps a request waiting for KV space
    if (reserved_blocks_ + need > eng_.total_blocks()) return;
    const int slot = eng_.allocate_slot();
    if (slot < 0) return;
    if (!eng_.reserve(slot, static_cast<int64_t>(head.req.prompt.size()) + head.req.max_new_tokens)) {
      eng_.free_slot(slot);
      return;
    }
    auto s = std::move(queue_.front());
    queue_.pop_front();
    s->slot = slot;
    s->reserved_blocks = need;
    s->t_admit = now();
    reserved_blocks_ += need;
    prefilling_.push_back(std::move(s));
  }
}

// mu_ held on entry and exit; released around the engine call
void BatchScheduler::run_prefill() {
  std::vector<PrefillItem> items;
  std::vector<Seq*> who;
  int budget = opt_.prefill_token_budget;
  for (auto& sp : prefilling_) {
    if (budget <= 0) break;
    Seq& s = *sp;
    if (s.cancelled) continue;
    const int64_t left = static_cast<int64_t>(s.req.prompt.size()) - s.prefilled;
    const int take = static_cast<int>(std::min<int64_t>({left, budget, opt_.prefill_chunk_tokens}));
    if (take <= 0) continue;
    PrefillItem it;
    it.slot = s.slot;
    it.position = s.prefilled;
    it.tokens.assign(s.req.prompt.begin() + s.prefilled, s.req.prompt.begin() + s.prefilled + take);
    it.last_chunk = (s.prefilled + take == static_cast<int64_t>(s.req.prompt.size()));
    items.push_back(std::move(it));
    who.push_back(&s);
    budget -= take;
  }
  if (items.empty()) return;
  StepResult res;
  std::string err;
  mu_.unlock();
  try { res = eng_.batch_prefill(items); } catch (const std::exception& e) { err = e.what(); }
  mu_.lock();
  for (size_t i = 0; i < who.size(); ++i) {
    Seq& s = *who[i];
    if (!err.empty() || res.next_tokens.size() != who.size()) { s.cancelled = true; s.out.clear(); s.last_token = -2; continue; }
    s.prefilled += static_cast<int64_t>(items[i].tokens.size());
    stats_.prefill_tokens += items[i].tokens.size();
    if (items[i].last_chunk) {
      s.last_token = res.next_tokens[i];
      s.t_first = now();
    }
  }
  // move finished prefills to the decode set (or finish them); drop failures
  std::vector<std::unique_ptr<Seq>> still;
  for (auto& sp : prefilling_) {
    Seq& s = *sp;
    if (s.last_token == -2) { finish(std::move(sp), "error", err.empty() ? "engine returned a malformed batch" : err); continue; }
    if (s.cancelled) { finish(std::move(sp), "cancelled"); continue; }
    if (s.prefilled < static_cast<int64_t>(s.req.prompt.size())) { still.push_back(std::move(sp)); continue; }
    // first generated token belongs to prefill
    const bool eos = s.req.stop_on_eos && eng_.is_eos(s.last_token);
    if (!eos) s.out.push_back(s.last_token);
    if (eos) finish(std::move(sp), "stop");
    else if (static_cast<int>(s.out.size()) >= s.req.max_new_tokens) finish(std::move(sp), "length");
    else decoding_.push_back(std::move(sp));
  }
  prefilling_ = std::move(still);
  cv_done_.notify_all();
}

void BatchScheduler::run_decode() {
  // drop cancelled sequences first
  {
    std::vector<std::unique_ptr<Seq>> keep;
    for (auto& sp : decoding_) {
      if (sp->cancelled) finish(std::move(sp), "cancelled");
      else keep.push_back(std::move(sp));
    }
    decoding_ = std::move(keep);
  }
  if (decoding_.empty()) return;
  std::vector<int> slots;
  std::vector<int32_t> toks;
  for (auto& sp : decoding_) { slots.push_back(sp->slot); toks.push_back(sp->last_token); }
  StepResult res;
  std::string err;
  mu_.unlock();
  try { res = eng_.batch_decode(slots, toks); } catch (const std::exception& e) { err = e.what(); }
  mu_.lock();
  std::vector<std::unique_ptr<Seq>> keep;
  for (size_t i = 0; i < decoding_.size(); ++i) {
    auto& sp = decoding_[i];
    Seq& s = *sp;
    if (!err.empty() || res.next_tokens.size() != slots.size()) { finish(std::move(sp), "error", err.empty() ? "engine returned a malformed batch" : err); continue; }
    const int32_t t = res.next_tokens[i];
    ++stats_.decode_tokens;
    if (s.req.stop_on_eos && eng_.is_eos(t)) { finish(std::move(sp), "stop"); continue; }
    s.out.push_back(t);
    s.last_token = t;
    if (static_cast<int>(s.out.size()) >= s.req.max_new_tokens) { finish(std::move(sp), "length"); continue; }
    if (s.cancelled) { finish(std::move(sp), "cancelled"); continue; }
    keep.push_back(std::move(sp));
  }
  decoding_ = std::move(keep);
  cv_done_.notify_all();
}

bool BatchScheduler::round() {
  std::unique_lock<std::mutex> g(mu_);
  if (queue_.empty() && prefilling_.empty() && decoding_.empty()) return false;
  ++stats_.rounds;
  if (opt_.decode_first) run_decode();
  admit();
  run_prefill();
  if (!opt_.decode_first) run_decode();
  return true;
}

bool BatchScheduler::step() { return round(); }

void BatchScheduler::loop() {
  while (!stop_.load()) {
    if (!round()) {
      std::unique_lock<std::mutex> g(mu_);
      cv_work_.wait_for(g, std::chrono::milliseconds(50), [this] {
        return stop_.load() || !queue_.empty() || !prefilling_.empty() || !decoding_.empty();
      });
    }
  }
}

}  // namespace pocket
