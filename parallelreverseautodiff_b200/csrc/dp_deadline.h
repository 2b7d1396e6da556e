// Host-side deadline for a collective that another rank may never join.
//
// The managed visitor bounds every wait on a sibling task with TimeoutInMinutes and queues an
// exception when it runs out (src/RMAD/OperationNeuralNetworkVisitor.cs:27,79-90,264-270).  The
// data-parallel path needs the same property between processes: a rank that died or never arrived
// must not leave the others blocked inside a collective for ever.  Nothing here touches a GPU: the
// loop polls two host-side questions ("has the communication stream reached my marker?", "has the
// communicator recorded an error?") until a deadline, then asks for the communicator to be aborted.
// It is a header of plain C++ so that it can be exercised with threads standing in for ranks.
#pragma once

#include <chrono>
#include <thread>

namespace prad {

enum class WaitOutcome { Done = 0, AsyncError = 1, TimedOut = 2 };

// done():  true once everything enqueued before the marker has completed (cudaEventQuery == success)
// error(): true if the communicator reports an asynchronous error (ncclCommGetAsyncError != success)
// abort(): called exactly once, on AsyncError or TimedOut, before returning (ncclCommAbort)
// The poll interval starts at 20 us and doubles up to 2 ms, so a collective that completes in time
// costs a handful of polls and a dead peer costs no measurable CPU.
template <class Done, class Error, class Abort>
WaitOutcome wait_with_deadline(Done done, Error error, Abort abort, double timeout_ms) {
  using clock = std::chrono::steady_clock;
  const auto t0 = clock::now();
  auto pause = std::chrono::microseconds(20);
  for (;;) {
    if (done()) return WaitOutcome::Done;
    if (error()) { abort(); return WaitOutcome::AsyncError; }
    const double waited = std::chrono::duration<double, std::milli>(clock::now() - t0).count();
    if (waited >= timeout_ms) {
      if (done()) return WaitOutcome::Done;   // completed while the clock was read
      abort();
      return WaitOutcome::TimedOut;
    }
    std::this_thread::sleep_for(pause);
    if (pause < std::chrono::microseconds(2000)) pause *= 2;
  }
}

}  // namespace prad
