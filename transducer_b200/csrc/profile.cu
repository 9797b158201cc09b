#include "profile.h"

#include <atomic>
#include <map>
#include <mutex>
#include <sstream>
#include <vector>

#include "common.cuh"

namespace tb200 {
namespace {

std::atomic<long long> g_launches{0};
std::atomic<bool> g_enabled{false};
std::mutex g_mu;

struct Record {
  std::string name;
  cudaEvent_t start, stop;
};
std::vector<Record> g_records;
constexpr size_t kMaxRecords = 1 << 16;

}  // namespace

ScopedKernel::ScopedKernel(const char* name, cudaStream_t stream) : slot_(-1), stream_(stream) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_enabled.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_records.size() >= kMaxRecords) return;
  Record r;
  r.name = name;
  if (cudaEventCreate(&r.start) != cudaSuccess) return;
  if (cudaEventCreate(&r.stop) != cudaSuccess) {
    cudaEventDestroy(r.start);
    return;
  }
  cudaEventRecord(r.start, stream);
  g_records.push_back(r);
  slot_ = (int)g_records.size() - 1;
}

ScopedKernel::~ScopedKernel() {
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lock(g_mu);
  if (slot_ < (int)g_records.size()) cudaEventRecord(g_records[slot_].stop, stream_);
}

long long launch_count() { return g_launches.load(); }

void profile_enable(bool on) { g_enabled.store(on); }

void profile_reset() {
  std::lock_guard<std::mutex> lock(g_mu);
  for (auto& r : g_records) {
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  g_records.clear();
}

std::string profile_report() {
  std::lock_guard<std::mutex> lock(g_mu);
  std::map<std::string, std::pair<long long, double>> agg;
  std::vector<std::string> order;
  for (auto& r : g_records) {
    if (cudaEventSynchronize(r.stop) != cudaSuccess) continue;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess) continue;
    if (!agg.count(r.name)) order.push_back(r.name);
    auto& a = agg[r.name];
    a.first += 1;
    a.second += ms;
  }
  std::ostringstream os;
  for (auto& n : order) os << n << ' ' << agg[n].first << ' ' << agg[n].second << '\n';
  return os.str();
}

}  // namespace tb200
