// Device status word shared by kernels and host code.
#pragma once
namespace b200 {

// Status word written by kernels whose waits are bounded or whose indices are
// checked.  0 = ok.  The host reads it after the launch when asked to.
enum KernelStatus : int {
  kOk = 0,
  kWaitTimeout = 1,      // an mbarrier / flag wait ran out of iterations
  kBadIndex = 2,         // an index (slot, block id, expert id) was out of range
  kBadShape = 3,
};

struct StatusWord {
  int code;
  int where;             // kernel-specific location id
  int expected;
  int observed;
};

}  // namespace b200
