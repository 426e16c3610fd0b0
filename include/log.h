// Log level switch of the operator API (reference: include/log.h:3-10).  `Log` is a global
// enum so that `generator.setLogMode(Log::Debug)` in user code keeps compiling.
#pragma once

enum Log { Debug = 0, Release = 1 };

namespace KernelCodeGen {

// Debug: dump() prints the IR and verifies it.  Release: dump() does nothing.
struct KCGLog {
  static Log level;
};

}  // namespace KernelCodeGen
