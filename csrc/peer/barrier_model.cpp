#include "barrier_model.h"

#include <atomic>
#include <chrono>
#include <memory>
#include <random>
#include <thread>
#include <vector>

namespace zx {

BarrierModelResult run_barrier_model(int ranks, int rounds, uint32_t start_epoch, uint64_t seed, int absent_rank,
                                     int absent_from_round, int64_t timeout_us) {
  // flags[r][t]: slot in rank r's flag buffer that rank t writes (the kernel's flags.p[r] + t)
  std::vector<std::unique_ptr<std::atomic<uint32_t>[]>> flags;
  for (int r = 0; r < ranks; ++r) {
    flags.emplace_back(new std::atomic<uint32_t>[ranks]);
    for (int t = 0; t < ranks; ++t) flags[r][t].store(start_epoch, std::memory_order_relaxed);
  }
  std::vector<int64_t> payload(ranks, -1);   // plain memory, ordered only by the barrier
  std::atomic<int64_t> violations{0}, timeouts{0};
  std::vector<std::atomic<int>> entered(ranks);
  for (auto& e : entered) e.store(-1);
  std::atomic<bool> give_up{false};
  std::vector<int> done(ranks, 0);
  auto body = [&](int rank) {
    std::mt19937_64 rng(seed * 1315423911ull + rank);
    auto jitter = [&]() {
      const int k = (int)(rng() % 4);
      if (k == 0) std::this_thread::yield();
      else if (k == 1) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 50));
    };
    uint32_t epoch = start_epoch;
    for (int round = 0; round < rounds && !give_up.load(); ++round) {
      if (rank == absent_rank && round >= absent_from_round) return;
      ++epoch;
      jitter();
      payload[rank] = round;                      // data written before the barrier
      entered[rank].store(round, std::memory_order_relaxed);
      // signal: one release store into every peer's buffer (the kernel does this from `ranks` threads)
      for (int t = 0; t < ranks; ++t) {
        jitter();
        flags[t][rank].store(epoch, std::memory_order_release);
      }
      // wait: acquire-poll my own buffer, one slot per peer, bounded
      bool ok = true;
      for (int t = 0; t < ranks && ok; ++t) {
        const auto t0 = std::chrono::steady_clock::now();
        while ((int32_t)(flags[rank][t].load(std::memory_order_acquire) - epoch) < 0) {
          if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(timeout_us)) { ok = false; break; }
          std::this_thread::yield();
        }
      }
      if (!ok) {                                   // the kernel reports a status and returns; so does the model
        timeouts.fetch_add(1);
        give_up.store(true);
        return;
      }
      // after the barrier: every rank must have entered this round and its payload must be visible
      for (int t = 0; t < ranks; ++t) {
        if (entered[t].load(std::memory_order_relaxed) < round) violations.fetch_add(1);
        if (payload[t] < round) violations.fetch_add(1);
      }
      ++done[rank];
      // second barrier of the round protects the payload cells from the next round's writes: reuse the
      // same protocol with the next epoch
      ++epoch;
      for (int t = 0; t < ranks; ++t) flags[t][rank].store(epoch, std::memory_order_release);
      for (int t = 0; t < ranks; ++t) {
        const auto t0 = std::chrono::steady_clock::now();
        while ((int32_t)(flags[rank][t].load(std::memory_order_acquire) - epoch) < 0) {
          if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(timeout_us)) { ok = false; break; }
          std::this_thread::yield();
        }
        if (!ok) break;
      }
      if (!ok) {
        timeouts.fetch_add(1);
        give_up.store(true);
        return;
      }
    }
  };
  std::vector<std::thread> threads;
  for (int r = 0; r < ranks; ++r) threads.emplace_back(body, r);
  for (auto& t : threads) t.join();
  int64_t min_done = rounds;
  for (int r = 0; r < ranks; ++r)
    if (r != absent_rank && done[r] < min_done) min_done = done[r];
  return {violations.load(), timeouts.load(), min_done};
}

}  // namespace zx
