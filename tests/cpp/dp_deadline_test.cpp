// CPU-only exercise of the deadline logic behind prad_dp_wait_host (csrc/dp_deadline.h), with threads
// standing in for ranks and a stub communicator: a collective "completes" when every rank has arrived.
// Prints one line per scenario: name, outcome (0 done, 1 async error, 2 timed out), abort calls, ms waited.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <thread>
#include <vector>

#include "../../parallelreverseautodiff_b200/csrc/dp_deadline.h"

struct StubComm {
  int world;
  std::atomic<int> arrived{0};
  std::atomic<bool> error{false};
  std::atomic<int> aborts{0};
  explicit StubComm(int w) : world(w) {}
  bool done() const { return arrived.load() >= world; }
};

static void scenario(const char* name, int world, int absent_rank, int late_ms, bool inject_error, double timeout_ms) {
  StubComm comm(world);
  std::vector<std::thread> ranks;
  std::vector<int> outcome(world, -1);
  std::vector<double> waited(world, 0.0);
  for (int r = 0; r < world; ++r) {
    ranks.emplace_back([&, r] {
      if (r == absent_rank) return;                         // this rank never joins the collective
      if (r == world - 1 && late_ms > 0) std::this_thread::sleep_for(std::chrono::milliseconds(late_ms));
      comm.arrived.fetch_add(1);
      if (inject_error && r == 0) comm.error.store(true);   // the stub's "ncclCommGetAsyncError != success"
      const auto t0 = std::chrono::steady_clock::now();
      const prad::WaitOutcome o = prad::wait_with_deadline(
          [&] { return comm.done(); }, [&] { return comm.error.load(); }, [&] { comm.aborts.fetch_add(1); }, timeout_ms);
      waited[r] = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
      outcome[r] = (int)o;
    });
  }
  for (auto& t : ranks) t.join();
  for (int r = 0; r < world; ++r)
    if (r != absent_rank) printf("%s rank=%d outcome=%d aborts=%d waited_ms=%.1f\n", name, r, outcome[r], comm.aborts.load(), waited[r]);
}

int main() {
  scenario("all_arrive", 4, -1, 0, false, 2000.0);
  scenario("one_late", 4, -1, 60, false, 2000.0);
  scenario("one_absent", 4, 2, 0, false, 150.0);
  scenario("async_error", 2, 1, 0, true, 2000.0);
  return 0;
}
