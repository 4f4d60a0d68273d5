// File-backed (NVMe) tier: asynchronous block reads/writes on worker threads.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace zxh {

// One file holding fixed-size slots; requests run on a small thread pool with pread/pwrite
// (O_DIRECT when the file system and the buffer alignment allow it, buffered otherwise).
class FileTier {
 public:
  FileTier(const std::string& path, int64_t slot_bytes, int64_t num_slots, int num_threads, bool try_direct);
  ~FileTier();
  FileTier(const FileTier&) = delete;
  FileTier& operator=(const FileTier&) = delete;

  // Returns a ticket; the buffer must stay valid until wait(ticket) returns.
  int64_t write_async(int64_t slot, const void* src, int64_t bytes);
  int64_t read_async(int64_t slot, void* dst, int64_t bytes);
  // Blocks until the request finished; returns 0 or a negative errno.
  int wait(int64_t ticket);
  void wait_all();
  bool direct() const { return direct_; }
  int64_t bytes_written() const { return bytes_written_; }
  int64_t bytes_read() const { return bytes_read_; }

 private:
  struct Req {
    int64_t ticket;
    bool is_write;
    int64_t slot;
    void* buf;
    int64_t bytes;
  };
  void worker();
  int fd_ = -1;
  bool direct_ = false;
  int64_t slot_bytes_, num_slots_;
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_req_, cv_done_;
  std::deque<Req> queue_;
  std::unordered_map<int64_t, int> done_;  // ticket -> status
  int64_t next_ticket_ = 1;
  int64_t in_flight_ = 0;
  bool stop_ = false;
  int64_t bytes_written_ = 0, bytes_read_ = 0;
};

}  // namespace zxh
