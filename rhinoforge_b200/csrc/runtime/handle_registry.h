// Process-wide table of native objects addressed by int64 handles.  Handles are
// issued monotonically and never reused, so a stale handle held by Python can
// only miss, never alias a newer object (same contract as the reference's
// ModelHandleRegistry, src/core/model_handle_registry.h:40-89).
#pragma once
#include <stdint.h>

#include <memory>
#include <mutex>
#include <unordered_map>

namespace rf {

template <typename T>
class HandleRegistry {
 public:
  int64_t insert(std::unique_ptr<T> obj) {
    std::lock_guard<std::mutex> g(mu_);
    const int64_t h = next_++;
    map_.emplace(h, std::shared_ptr<T>(std::move(obj)));
    return h;
  }
  std::shared_ptr<T> get(int64_t h) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(h);
    return it == map_.end() ? nullptr : it->second;
  }
  bool erase(int64_t h) {
    std::lock_guard<std::mutex> g(mu_);
    return map_.erase(h) > 0;
  }
  size_t size() {
    std::lock_guard<std::mutex> g(mu_);
    return map_.size();
  }

 private:
  std::mutex mu_;
  std::unordered_map<int64_t, std::shared_ptr<T>> map_;
  int64_t next_ = 1;
};

}  // namespace rf
