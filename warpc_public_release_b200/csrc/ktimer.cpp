// Kernel durations on the GPU's own clock, through CUPTI activity records
// (CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL, which does not serialise kernels): the measurement
// the reference publishes its numbers with (backend/node/ktrace.cpp:21-88, README.md:504-525 --
// there an injection library that reports at exit; here a small C ABI a harness drives, so
// several kernels can be compared inside one process and one warm GPU).
//
//   wk_begin()                      start recording
//   wk_end()                        flush and stop
//   wk_count(), wk_get(i, ...)      the records, in start order
//   wk_median(substr, last, ...)    median duration of the last `last` kernels whose name contains substr
#include <cupti.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace {
struct Rec {
  uint64_t start, end;
  std::string name;
};
std::vector<Rec> g_recs;
std::mutex g_mutex;
bool g_registered = false, g_on = false;

void CUPTIAPI buffer_requested(uint8_t** buffer, size_t* size, size_t* max_records) {
  *size = 4u << 20;
  *buffer = static_cast<uint8_t*>(aligned_alloc(8, *size));
  *max_records = 0;
}

void CUPTIAPI buffer_completed(CUcontext, uint32_t, uint8_t* buffer, size_t, size_t valid) {
  CUpti_Activity* rec = nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  while (valid > 0 && cuptiActivityGetNextRecord(buffer, valid, &rec) == CUPTI_SUCCESS) {
    if (rec->kind != CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL && rec->kind != CUPTI_ACTIVITY_KIND_KERNEL) continue;
    const auto* k = reinterpret_cast<const CUpti_ActivityKernel9*>(rec);
    g_recs.push_back({k->start, k->end, k->name ? k->name : "?"});
  }
  free(buffer);
}
}  // namespace

extern "C" int wk_begin() {
  if (!g_registered) {
    if (cuptiActivityRegisterCallbacks(buffer_requested, buffer_completed) != CUPTI_SUCCESS) return -1;
    g_registered = true;
  }
  if (!g_on) {
    if (cuptiActivityEnable(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL) != CUPTI_SUCCESS) return -2;
    g_on = true;
  }
  return 0;
}

extern "C" int wk_end() {
  if (!g_on) return 0;
  cuptiActivityFlushAll(1);
  cuptiActivityDisable(CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL);
  g_on = false;
  std::lock_guard<std::mutex> lock(g_mutex);
  std::sort(g_recs.begin(), g_recs.end(), [](const Rec& a, const Rec& b) { return a.start < b.start; });
  return 0;
}

extern "C" int wk_flush() {
  cuptiActivityFlushAll(1);
  std::lock_guard<std::mutex> lock(g_mutex);
  std::sort(g_recs.begin(), g_recs.end(), [](const Rec& a, const Rec& b) { return a.start < b.start; });
  return 0;
}

extern "C" void wk_clear() {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_recs.clear();
}

extern "C" int wk_count() {
  std::lock_guard<std::mutex> lock(g_mutex);
  return int(g_recs.size());
}

extern "C" int wk_get(int i, char* name, size_t cap, double* start_us, double* dur_us) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (i < 0 || size_t(i) >= g_recs.size()) return -1;
  const Rec& r = g_recs[size_t(i)];
  if (name && cap) {
    std::strncpy(name, r.name.c_str(), cap - 1);
    name[cap - 1] = 0;
  }
  if (start_us) *start_us = double(r.start) / 1e3;
  if (dur_us) *dur_us = double(r.end - r.start) / 1e3;
  return 0;
}

// Median (and min / max) duration in microseconds over the last `last` recorded kernels whose
// name contains `substr` (all of them when last <= 0).  Returns how many were used.
extern "C" int wk_median(const char* substr, int last, double* median_us, double* min_us, double* max_us) {
  std::lock_guard<std::mutex> lock(g_mutex);
  std::vector<double> d;
  for (const Rec& r : g_recs)
    if (!substr || !*substr || r.name.find(substr) != std::string::npos) d.push_back(double(r.end - r.start) / 1e3);
  if (last > 0 && d.size() > size_t(last)) d.erase(d.begin(), d.end() - last);
  if (d.empty()) return 0;
  std::sort(d.begin(), d.end());
  if (median_us) *median_us = d[d.size() / 2];
  if (min_us) *min_us = d.front();
  if (max_us) *max_us = d.back();
  return int(d.size());
}
