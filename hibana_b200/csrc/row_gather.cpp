// Host-side gather of fixed-size rows from a table sharded over many files (the n-gram "PLE" embedding table of the
// Flash-Next family: a few 160-byte rows per token out of a table far larger than GPU memory, living on NVMe).
//
// Pass 1 tries every row with preadv2(RWF_NOWAIT) on the calling thread: rows whose pages are in the page cache
// are copied at memory speed and cost no thread hop. Pass 2 hands the misses to a small pool of worker threads
// that issue blocking preads in parallel (NVMe queue depth = pool size). The destination can be pinned host memory,
// from where one async copy takes the batch to the GPU. No Python objects are touched, so the caller releases the
// GIL around the call. Reference counterpart: hibana/kernels/csrc/ple_gather.cpp (same two-pass scheme).
#include <atomic>
#include <condition_variable>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <string>
#include <sys/uio.h>
#include <thread>
#include <unistd.h>
#include <vector>

#include "hb_api.h"

namespace {

struct Job {
  int fd;
  int64_t offset;
  uint8_t* dst;
};

class Gatherer {
 public:
  Gatherer(int row_bytes, int64_t rows_per_shard, int threads) : row_bytes_(row_bytes), rows_per_shard_(rows_per_shard) {
    for (int i = 0; i < threads; ++i) workers_.emplace_back([this] { work(); });
  }
  ~Gatherer() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
    for (int fd : fds_) ::close(fd);
  }
  bool add_shard(const char* path) {
    const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return false;
    fds_.push_back(fd);
    return true;
  }
  // Returns rows read, or -(index + 1) of the first row that could not be read. `cold` counts pass-2 rows.
  int64_t gather(const int64_t* rows, int64_t n, uint8_t* dst, int64_t* cold) {
    std::vector<Job> misses;
    for (int64_t i = 0; i < n; ++i) {
      const int64_t r = rows[i];
      const int64_t shard = r / rows_per_shard_;
      if (r < 0 || shard >= static_cast<int64_t>(fds_.size())) return -(i + 1);
      Job j{fds_[shard], (r % rows_per_shard_) * row_bytes_, dst + i * row_bytes_};
      struct iovec iov{j.dst, static_cast<size_t>(row_bytes_)};
      const ssize_t got = ::preadv2(j.fd, &iov, 1, j.offset, RWF_NOWAIT);
      if (got != row_bytes_) misses.push_back(j);   // EAGAIN (not cached), short read, or no RWF_NOWAIT support
    }
    if (cold) *cold = static_cast<int64_t>(misses.size());
    if (misses.empty()) return n;
    std::atomic<int64_t> failed{0};
    {
      std::unique_lock<std::mutex> lk(mu_);
      pending_ = static_cast<int64_t>(misses.size());
      jobs_ = misses.data();
      next_ = 0;
      total_ = static_cast<int64_t>(misses.size());
      failed_ = &failed;
    }
    cv_.notify_all();
    // the caller works too
    run_jobs();
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [this] { return pending_ == 0; });
    jobs_ = nullptr;
    return failed.load() ? -1 : n;
  }

 private:
  void run_jobs() {
    for (;;) {
      int64_t i;
      Job j;
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (jobs_ == nullptr || next_ >= total_) return;
        i = next_++;
        j = jobs_[i];
      }
      int64_t off = 0;
      bool ok = true;
      while (off < row_bytes_) {
        const ssize_t got = ::pread(j.fd, j.dst + off, row_bytes_ - off, j.offset + off);
        if (got <= 0) {
          if (got < 0 && errno == EINTR) continue;
          ok = false;
          break;
        }
        off += got;
      }
      std::lock_guard<std::mutex> lk(mu_);
      if (!ok) failed_->fetch_add(1);
      if (--pending_ == 0) done_cv_.notify_all();
    }
  }
  void work() {
    for (;;) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || (jobs_ != nullptr && next_ < total_); });
        if (stop_) return;
      }
      run_jobs();
    }
  }

  const int row_bytes_;
  const int64_t rows_per_shard_;
  std::vector<int> fds_;
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  bool stop_ = false;
  Job* jobs_ = nullptr;
  int64_t next_ = 0, total_ = 0, pending_ = 0;
  std::atomic<int64_t>* failed_ = nullptr;
};

}  // namespace

extern "C" {

void* hb_rows_open(int row_bytes, long long rows_per_shard, int threads) {
  if (row_bytes <= 0 || rows_per_shard <= 0 || threads < 0 || threads > 256) return nullptr;
  return new Gatherer(row_bytes, rows_per_shard, threads);
}
int hb_rows_add_shard(void* g, const char* path) { return static_cast<Gatherer*>(g)->add_shard(path) ? 0 : 1; }
long long hb_rows_gather(void* g, const long long* rows, long long n, void* dst, long long* cold) {
  int64_t c = 0;
  const int64_t r = static_cast<Gatherer*>(g)->gather(reinterpret_cast<const int64_t*>(rows), n,
                                                      static_cast<uint8_t*>(dst), &c);
  if (cold) *cold = c;
  return r;
}
void hb_rows_close(void* g) { delete static_cast<Gatherer*>(g); }

}  // extern "C"
