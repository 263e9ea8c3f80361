// Abstract slot / paged-KV / batch interface the scheduler drives.
// (Role of cpp_engine/include/inference_engine.hpp:126-181; a concrete engine is supplied by the
// native runtime or, from Python, through a trampoline in the pybind module.)
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace pocket {

struct PrefillItem {
  int slot = -1;
  std::vector<int32_t> tokens;   // the part of the prompt to run in this call
  int64_t position = 0;          // context position of tokens[0]
  bool last_chunk = true;        // the call must return the next token only when true
};

struct StepResult {
  std::vector<int32_t> next_tokens;  // one per item (prefill: -1 when !last_chunk)
};

class InferenceEngine {
 public:
  virtual ~InferenceEngine() = default;
  virtual int max_slots() const = 0;
  virtual int block_tokens() const = 0;
  virtual int total_blocks() const = 0;
  virtual int64_t max_context() const = 0;
  virtual int allocate_slot() = 0;                                   // -1 when none is free
  virtual void free_slot(int slot) = 0;
  // Reserve KV blocks so `slot` can hold `tokens` tokens; false if the pool cannot supply them.
  virtual bool reserve(int slot, int64_t tokens) = 0;
  virtual StepResult batch_prefill(const std::vector<PrefillItem>& items) = 0;
  virtual StepResult batch_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens) = 0;
  virtual bool is_eos(int32_t token) const = 0;
  // Number of token ids the model knows (ids are 0 .. vocab_size - 1); 0 when the engine cannot say.  Front ends use it
  // to refuse a request whose token ids the model has no row for, before anything reaches a device.
  virtual int64_t vocab_size() const { return 0; }
};

}  // namespace pocket
