// Belady MIN over byte-sized blocks: on a miss that does not fit, evict the resident block whose
// next use lies farthest in the future (never-used-again first). The access order of ring
// attention is known before the step starts, which is what makes the offline policy usable online.
// The reference's BeladyApproxCache counts items, not bytes, and relies on the caller to feed it
// next-use times (zenyx/streaming/belady.py:8-58).
#include "belady_min.h"

#include <algorithm>
#include <list>
#include <set>
#include <unordered_map>

namespace zxh {

BeladyResult belady_min(const std::vector<int64_t>& ids, const std::vector<int64_t>& size_of, int64_t capacity) {
  const int64_t n = (int64_t)ids.size();
  const int64_t never = n + 1;
  BeladyResult r;
  r.hit.assign(n, 0);
  r.evicted.assign(n, {});
  r.next_use.assign(n, -1);
  std::vector<int64_t> last(size_of.size(), -1);
  for (int64_t i = n - 1; i >= 0; --i) {
    r.next_use[i] = last[ids[i]];
    last[ids[i]] = i;
  }
  // resident set ordered by next use (farthest last); key = (next use, id)
  std::set<std::pair<int64_t, int64_t>> by_next;
  std::vector<int64_t> key_of(size_of.size(), -1);  // current next-use key of a resident block, -1 if absent
  int64_t resident = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    const int64_t nu = r.next_use[i] < 0 ? never : r.next_use[i];
    if (key_of[id] >= 0) {
      r.hit[i] = 1;
      ++r.hits;
      by_next.erase({key_of[id], id});
      key_of[id] = nu;
      by_next.insert({nu, id});
      continue;
    }
    ++r.misses;
    const int64_t sz = size_of[id];
    r.bytes_loaded += sz;
    if (sz > capacity) {
      ++r.bypassed;
      continue;
    }
    while (resident + sz > capacity && !by_next.empty()) {
      auto it = std::prev(by_next.end());
      // MIN: if the incoming block is itself the farthest, keeping it would be the worst choice
      if (it->first < nu) {
        break;
      }
      const int64_t victim = it->second;
      by_next.erase(it);
      key_of[victim] = -1;
      resident -= size_of[victim];
      r.bytes_evicted += size_of[victim];
      r.evicted[i].push_back(victim);
    }
    if (resident + sz > capacity) {
      ++r.bypassed;  // everything resident is needed sooner: stream this block through without keeping it
      continue;
    }
    resident += sz;
    key_of[id] = nu;
    by_next.insert({nu, id});
    r.peak_resident_bytes = std::max(r.peak_resident_bytes, resident);
  }
  return r;
}

BeladyResult lru_trace(const std::vector<int64_t>& ids, const std::vector<int64_t>& size_of, int64_t capacity) {
  const int64_t n = (int64_t)ids.size();
  BeladyResult r;
  r.hit.assign(n, 0);
  r.evicted.assign(n, {});
  r.next_use.assign(n, -1);
  std::list<int64_t> order;  // front = most recent
  std::unordered_map<int64_t, std::list<int64_t>::iterator> where;
  int64_t resident = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    auto it = where.find(id);
    if (it != where.end()) {
      r.hit[i] = 1;
      ++r.hits;
      order.erase(it->second);
      order.push_front(id);
      where[id] = order.begin();
      continue;
    }
    ++r.misses;
    const int64_t sz = size_of[id];
    r.bytes_loaded += sz;
    if (sz > capacity) {
      ++r.bypassed;
      continue;
    }
    while (resident + sz > capacity && !order.empty()) {
      const int64_t victim = order.back();
      order.pop_back();
      where.erase(victim);
      resident -= size_of[victim];
      r.bytes_evicted += size_of[victim];
      r.evicted[i].push_back(victim);
    }
    resident += sz;
    order.push_front(id);
    where[id] = order.begin();
    r.peak_resident_bytes = std::max(r.peak_resident_bytes, resident);
  }
  return r;
}

}  // namespace zxh
