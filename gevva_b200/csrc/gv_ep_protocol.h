// The cross-rank barrier of the expert-parallel path as a state machine that compiles for the
// device (flags in peer memory, SM cycle counter) and for the host (atomics, steady clock), so
// that the protocol, including what happens when a rank never arrives, is tested with threads on
// a CPU and no GPU is ever made to wait for a rank that is not coming.
//
// Every rank owns `world` flags.  In barrier number `epoch` (1, 2, ...) rank r stores `epoch`
// into flag r of every rank and then waits until each of its own flags has reached `epoch`
// (flags only grow, so a rank that is late for one barrier and catches up later finds the others'
// newer values acceptable).  The wait is bounded: when Port::expired() says so the function
// returns false and the caller records a timeout; nothing spins forever.
//
// Port supplies the memory and the clock:
//   void publish(int peer, int slot, int value)   release-store into flag `slot` of rank `peer`
//   int  observe(int slot)                        acquire-load of this rank's own flag `slot`
//   void start_clock(); bool expired(); void pause();
#pragma once

#if defined(__CUDACC__)
#define GV_HOST_DEVICE __host__ __device__
#else
#define GV_HOST_DEVICE
#endif

namespace gv {

// One lane's share of a barrier: announce to rank `lane`, then wait for rank `lane`'s announcement.
// On the device 32 lanes run this side by side; on the host a loop over the lanes does the same
// (all announcements first, then the waits).
template <class Port>
GV_HOST_DEVICE inline void ep_barrier_announce(Port& port, int rank, int lane, int epoch) {
  port.publish(lane, rank, epoch);
}

template <class Port>
GV_HOST_DEVICE inline bool ep_barrier_await(Port& port, int lane, int epoch) {
  port.start_clock();
  for (;;) {
    if (port.observe(lane) - epoch >= 0) return true;
    if (port.expired()) return false;
    port.pause();
  }
}

}  // namespace gv
