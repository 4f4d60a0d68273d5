// NVMe tier of the KV tiering manager. The reference's "T2" is a Python dict of CPU tensors with
// no file I/O (zenyx/streaming/kv_tiering.py:23,29); this is an actual file tier.
#include "tier_engine.h"

#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <stdexcept>
#include <unistd.h>

namespace zxh {

FileTier::FileTier(const std::string& path, int64_t slot_bytes, int64_t num_slots, int num_threads, bool try_direct)
    : slot_bytes_(slot_bytes), num_slots_(num_slots) {
  if (slot_bytes <= 0 || num_slots <= 0) throw std::runtime_error("FileTier: bad geometry");
  if (try_direct && slot_bytes % 4096 == 0) {
    fd_ = ::open(path.c_str(), O_RDWR | O_CREAT | O_DIRECT, 0600);
    direct_ = fd_ >= 0;
  }
  if (fd_ < 0) fd_ = ::open(path.c_str(), O_RDWR | O_CREAT, 0600);
  if (fd_ < 0) throw std::runtime_error("FileTier: cannot open " + path + ": " + std::strerror(errno));
  if (::ftruncate(fd_, slot_bytes * num_slots) != 0) {
    const std::string msg = std::strerror(errno);
    ::close(fd_);
    throw std::runtime_error("FileTier: cannot size the backing file: " + msg);
  }
  if (num_threads < 1) num_threads = 1;
  for (int i = 0; i < num_threads; ++i) threads_.emplace_back([this] { worker(); });
}

FileTier::~FileTier() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_req_.notify_all();
  for (auto& t : threads_) t.join();
  if (fd_ >= 0) ::close(fd_);
}

int64_t FileTier::write_async(int64_t slot, const void* src, int64_t bytes) {
  if (slot < 0 || slot >= num_slots_ || bytes > slot_bytes_) throw std::runtime_error("FileTier: slot out of range");
  std::lock_guard<std::mutex> lk(mu_);
  const int64_t t = next_ticket_++;
  queue_.push_back({t, true, slot, const_cast<void*>(src), bytes});
  ++in_flight_;
  cv_req_.notify_one();
  return t;
}

int64_t FileTier::read_async(int64_t slot, void* dst, int64_t bytes) {
  if (slot < 0 || slot >= num_slots_ || bytes > slot_bytes_) throw std::runtime_error("FileTier: slot out of range");
  std::lock_guard<std::mutex> lk(mu_);
  const int64_t t = next_ticket_++;
  queue_.push_back({t, false, slot, dst, bytes});
  ++in_flight_;
  cv_req_.notify_one();
  return t;
}

void FileTier::worker() {
  for (;;) {
    Req rq;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_req_.wait(lk, [this] { return stop_ || !queue_.empty(); });
      if (queue_.empty()) return;
      rq = queue_.front();
      queue_.pop_front();
    }
    int status = 0;
    int64_t done = 0;
    const bool aligned = (reinterpret_cast<uintptr_t>(rq.buf) % 4096 == 0) && (rq.bytes % 4096 == 0);
    if (direct_ && !aligned) status = -EINVAL;  // O_DIRECT needs 4 KiB-aligned buffers and sizes
    while (status == 0 && done < rq.bytes) {
      const off_t off = (off_t)(rq.slot * slot_bytes_ + done);
      const ssize_t n = rq.is_write ? ::pwrite(fd_, static_cast<char*>(rq.buf) + done, rq.bytes - done, off)
                                    : ::pread(fd_, static_cast<char*>(rq.buf) + done, rq.bytes - done, off);
      if (n < 0) {
        if (errno == EINTR) continue;
        status = -errno;
      } else if (n == 0) {
        status = -EIO;
      } else {
        done += n;
      }
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      done_[rq.ticket] = status;
      --in_flight_;
      if (status == 0) (rq.is_write ? bytes_written_ : bytes_read_) += rq.bytes;
    }
    cv_done_.notify_all();
  }
}

int FileTier::wait(int64_t ticket) {
  std::unique_lock<std::mutex> lk(mu_);
  cv_done_.wait(lk, [&] { return done_.count(ticket) > 0; });
  const int st = done_[ticket];
  done_.erase(ticket);
  return st;
}

void FileTier::wait_all() {
  std::unique_lock<std::mutex> lk(mu_);
  cv_done_.wait(lk, [&] { return in_flight_ == 0; });
}

}  // namespace zxh
