// Row-parallel driver of the CPU checkers. TEST INFRASTRUCTURE ONLY.
//
// ForRows(rows, threads, fn) splits [0, rows) into `threads` contiguous chunks and runs fn(begin, end) on each.
// The reference threads only its MatVec (src/model/cpu_ops.cpp:120-131; its trainer splits norm rows the same
// way, src/train/last_k.cpp:41-52), so this driver is ours. Workers are persistent: a benchmark step makes
// several hundred operator calls, and spawning and joining a thread per chunk per call cost a fifth of the
// step. The calling thread takes the first chunk itself. One call at a time (the checkers are driven from one
// Python thread); a nested or concurrent call falls back to running inline.
#ifndef HALO_ORACLE_ROW_POOL_HPP_
#define HALO_ORACLE_ROW_POOL_HPP_

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace halo_oracle {

class RowPool {
 public:
  static RowPool& Instance() {
    static RowPool* pool = new RowPool;  // never destroyed: workers may outlive static destructors
    return *pool;
  }

  void Run(std::size_t rows, int threads, const std::function<void(std::size_t, std::size_t)>& fn) {
    if (threads <= 1 || rows < 2) {
      fn(0, rows);
      return;
    }
    std::unique_lock<std::mutex> call(call_mutex_, std::try_to_lock);
    if (!call.owns_lock()) {  // nested or concurrent use
      fn(0, rows);
      return;
    }
    const std::size_t nt = std::min<std::size_t>(static_cast<std::size_t>(threads), rows);
    const std::size_t chunk = (rows + nt - 1) / nt;
    const std::size_t chunks = (rows + chunk - 1) / chunk;
    Grow(chunks - 1);
    {
      std::lock_guard<std::mutex> lock(mutex_);
      fn_ = &fn;
      rows_ = rows;
      chunk_ = chunk;
      active_ = chunks - 1;   // workers 0 .. chunks - 2 take chunks 1 .. chunks - 1
      pending_ = chunks - 1;
      ++generation_;
    }
    wake_.notify_all();
    fn(0, std::min(rows, chunk));
    std::unique_lock<std::mutex> lock(mutex_);
    done_.wait(lock, [this] { return pending_ == 0; });
    fn_ = nullptr;
  }

 private:
  void Grow(std::size_t want) {
    while (workers_.size() < want) {
      const std::size_t id = workers_.size();
      workers_.emplace_back([this, id] { Work(id); });
      workers_.back().detach();
    }
  }

  void Work(std::size_t id) {
    std::size_t seen = 0;
    for (;;) {
      const std::function<void(std::size_t, std::size_t)>* fn = nullptr;
      std::size_t begin = 0, end = 0;
      {
        std::unique_lock<std::mutex> lock(mutex_);
        wake_.wait(lock, [&] { return generation_ != seen; });
        seen = generation_;
        if (id >= active_) continue;
        fn = fn_;
        begin = (id + 1) * chunk_;
        end = std::min(rows_, begin + chunk_);
      }
      (*fn)(begin, end);
      {
        std::lock_guard<std::mutex> lock(mutex_);
        --pending_;
      }
      done_.notify_one();
    }
  }

  std::mutex call_mutex_, mutex_;
  std::condition_variable wake_, done_;
  std::vector<std::thread> workers_;
  const std::function<void(std::size_t, std::size_t)>* fn_ = nullptr;
  std::size_t rows_ = 0, chunk_ = 0, active_ = 0, pending_ = 0, generation_ = 0;
};

template <typename Fn>
void ForRows(std::size_t rows, int threads, Fn fn) {
  RowPool::Instance().Run(rows, threads, std::function<void(std::size_t, std::size_t)>(fn));
}

}  // namespace halo_oracle

#endif  // HALO_ORACLE_ROW_POOL_HPP_
